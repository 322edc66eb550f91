"""JSON / HTML string helpers of the chart package (legacy/src/momijo/visual/core/core.mojo:6-154,
core/echarts_core.mojo:7-22). Everything in ``momijo_b200.visual`` produces ECharts option JSON or a
self-contained HTML page as text; nothing is rendered here."""
from __future__ import annotations

import html as _html
import json
import math
import os
from typing import Iterable, Sequence

ECHARTS_CDN = "https://cdn.jsdelivr.net/npm/echarts@5/dist/echarts.min.js"
ECHARTS_GL_CDN = "https://cdn.jsdelivr.net/npm/echarts-gl@2/dist/echarts-gl.min.js"
WORDCLOUD_CDN = "https://cdn.jsdelivr.net/npm/echarts-wordcloud@2/dist/echarts-wordcloud.min.js"
WORLD_MAP_CDN = "https://cdn.jsdelivr.net/npm/echarts@4.9.0/map/js/world.js"


def _num(x) -> str:
    x = float(x)
    if math.isnan(x) or math.isinf(x):
        return "null"
    return repr(int(x)) if x == int(x) and abs(x) < 1e15 else repr(x)


def dumps(obj) -> str:
    """Compact JSON; NaN / inf become null so that the page's ``JSON.parse`` accepts it."""
    def clean(o):
        if isinstance(o, float):
            return None if (math.isnan(o) or math.isinf(o)) else o
        if isinstance(o, dict):
            return {str(k): clean(v) for k, v in o.items()}
        if isinstance(o, (list, tuple)):
            return [clean(v) for v in o]
        if hasattr(o, "tolist"):
            return clean(o.tolist())
        return o
    return json.dumps(clean(obj), separators=(",", ":"), ensure_ascii=False)


def _single_to_double_quoted(s: str) -> str:
    """Rewrite a JavaScript-style fragment with single-quoted strings as JSON: quotes are swapped, embedded double
    quotes escaped, ``\\'`` unescaped."""
    out, i, n = [], 0, len(s)
    while i < n:
        ch = s[i]
        if ch == '"':                                   # already a JSON string: copy through
            j = i + 1
            while j < n and s[j] != '"':
                j += 2 if s[j] == "\\" else 1
            out.append(s[i:j + 1])
            i = j + 1
        elif ch == "'":
            j, buf = i + 1, []
            while j < n and s[j] != "'":
                if s[j] == "\\" and j + 1 < n:
                    buf.append("'" if s[j + 1] == "'" else s[j:j + 2])
                    j += 2
                else:
                    buf.append('\\"' if s[j] == '"' else s[j])
                    j += 1
            out.append('"' + "".join(buf) + '"')
            i = j + 1
        else:
            out.append(ch)
            i += 1
    return "".join(out)


def loads(s: str):
    """Parse a JSON fragment. The reference writes its fragments with single quotes (``{ 'type':'value' }``), so when
    strict JSON fails the single-quoted form is accepted too."""
    try:
        return json.loads(s)
    except json.JSONDecodeError:
        return json.loads(_single_to_double_quoted(s))


def json_string(s: str) -> str:
    return json.dumps(str(s), ensure_ascii=False)


def json_array_str(items: Iterable[str]) -> str:
    """Join already-serialised JSON fragments into an array."""
    return "[" + ",".join(items) + "]"


def json_number_array(xs: Sequence[float]) -> str:
    return "[" + ",".join(_num(x) for x in xs) + "]"


json_array_f64 = json_number_array


def json_string_array(xs: Sequence[str]) -> str:
    return "[" + ",".join(json_string(x) for x in xs) + "]"


def escape_html(s: str) -> str:
    return _html.escape(str(s), quote=True)


def echarts_html(option_json: str, title: str = "Chart", width_px: int = 960, height_px: int = 540,
                 theme: str = "", include_gl: bool = False, include_world_map: bool = False,
                 include_wordcloud_plugin: bool = False, pre_init_js: str = "", full_page: bool = False) -> str:
    """A standalone page that loads ECharts from its CDN and applies ``option_json``."""
    scripts = [ECHARTS_CDN]
    if include_gl:
        scripts.append(ECHARTS_GL_CDN)
    if include_world_map:
        scripts.append(WORLD_MAP_CDN)
    if include_wordcloud_plugin:
        scripts.append(WORDCLOUD_CDN)
    tags = "".join(f'<script src="{u}"></script>' for u in scripts)
    size = "width:100vw;height:100vh" if full_page else f"width:{int(width_px)}px;height:{int(height_px)}px"
    theme_arg = f", {json_string(theme)}" if theme else ""
    return ("<!doctype html><html><head><meta charset=\"utf-8\">"
            f"<meta name=\"viewport\" content=\"width=device-width,initial-scale=1\"><title>{escape_html(title)}</title>"
            f"{tags}<style>html,body{{margin:0;padding:0}}#chart{{{size}}}</style></head><body>"
            "<div id=\"chart\"></div><script>"
            f"{pre_init_js}\nvar chart = echarts.init(document.getElementById('chart'){theme_arg});\n"
            f"var option = {option_json};\nchart.setOption(option);\n"
            "window.addEventListener('resize', function(){chart.resize();});</script></body></html>")


def write_text(path: str, text: str) -> bool:
    try:
        d = os.path.dirname(os.path.abspath(path))
        os.makedirs(d, exist_ok=True)
        with open(path, "w", encoding="utf-8") as f:
            f.write(text)
        return True
    except OSError:
        return False
