"""HTML output (legacy/src/momijo/visual/html/html_viewer.mojo:24-125, html/preview.mojo:9-67). The
reference opens the page in a browser through Python interop and snapshots it with Puppeteer; this
machine class has neither a browser nor a display, so pages are written to disk and ``open_in_browser``
only reports the path."""
from __future__ import annotations

import os

from .core import echarts_html, write_text


def open_in_browser(file_path: str) -> bool:
    print("open_in_browser: no browser here; page is at", os.path.abspath(file_path))
    return False


def write_preview_html(html: str, save: bool, out_path: str) -> str:
    if save:
        write_text(out_path, html)
        return os.path.abspath(out_path)
    return ""


def render_html(option_json: str, title: str = "momijo - ECharts", width_px: int = 960, height_px: int = 540,
                include_world_map: bool = False, save: bool = True, auto_open: bool = False,
                out_path: str = "chart.html", full_page: bool = False, include_gl: bool = False,
                pre_init_js: str = "", include_wordcloud_plugin: bool = False) -> str:
    page = echarts_html(option_json, title, width_px, height_px, include_gl=include_gl,
                        include_world_map=include_world_map, include_wordcloud_plugin=include_wordcloud_plugin,
                        pre_init_js=pre_init_js, full_page=full_page)
    path = write_preview_html(page, save, out_path)
    if auto_open and path:
        open_in_browser(path)
    return page


def _px(v, default: int) -> int:
    """``960``, ``"480px"`` -> pixels; percentages and anything else fall back to ``default``."""
    if isinstance(v, (int, float)):
        return int(v)
    s = str(v).strip().lower()
    return int(float(s[:-2])) if s.endswith("px") and s[:-2].replace(".", "", 1).isdigit() else default


def render_echarts(opts_json: str, outfile: str, title: str = "Chart", width_px=960, height_px=540,
                   theme: str = "", auto_open: bool = False, include_gl: bool = False, *ref_tail) -> bool:
    """Write a standalone page. The reference's argument order ``(opts_json, outfile, title, div_id, width, height,
    renderer, theme, enable_download, auto_open)`` (legacy/src/momijo/visual/html/html_viewer.mojo:24-35) is recognised
    by a string in the fourth position (the div id): CSS sizes are converted to pixels and the page is never opened
    here (there is no browser on a server)."""
    if isinstance(width_px, str) and not width_px.strip().lower().endswith(("px", "%")) and not width_px.isdigit():
        width, height = height_px, theme                      # (div_id, width, height, renderer, theme, ...)
        theme = ref_tail[0] if ref_tail else ""
        width_px, height_px, auto_open, include_gl = _px(width, 960), _px(height, 480), False, False
    else:
        width_px, height_px = _px(width_px, 960), _px(height_px, 540)
    ok = write_text(outfile, echarts_html(opts_json, title, width_px, height_px, theme=theme, include_gl=include_gl))
    if ok and auto_open:
        open_in_browser(outfile)
    return ok


def preview(option_json: str, title: str = "ECharts Demo", width_px: int = 960, height_px: int = 750,
            out_path: str = "chart.html", auto_open: bool = False, full_page: bool = True, include_gl: bool = False,
            pre_init_js: str = "", include_wordcloud_plugin: bool = False) -> str:
    return render_html(option_json, title=title, width_px=width_px, height_px=height_px, include_world_map=False,
                       save=True, auto_open=auto_open, out_path=out_path, full_page=full_page, include_gl=include_gl,
                       pre_init_js=pre_init_js, include_wordcloud_plugin=include_wordcloud_plugin)
