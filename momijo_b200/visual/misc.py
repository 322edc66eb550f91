"""Per-chart option builders, the ``Figure`` record, numeric helpers (histogram, KDE, marching squares),
themes and the exporter registry (legacy/src/momijo/visual/misc/*.mojo, plotting/echarts_exporter.mojo).
The reference emits JavaScript object literals with unquoted keys; these emit strict JSON, which ECharts
accepts just the same and which can be parsed back in tests."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

from .core import dumps, echarts_html, escape_html, write_text, ECHARTS_CDN


@dataclass
class Figure:
    _title: str = ""
    _y_name: str = ""
    _w: int = 960
    _h: int = 540
    _xs: List[str] = field(default_factory=list)
    _ys: List[List[float]] = field(default_factory=list)
    _names: List[str] = field(default_factory=list)

    def title(self): return self._title
    def y_label(self): return self._y_name
    def width_px(self): return self._w
    def height_px(self): return self._h
    def to_line_triplet(self): return (list(self._xs), [list(y) for y in self._ys], list(self._names))


def title(fig: Figure) -> str: return fig.title()
def y_label(fig: Figure) -> str: return fig.y_label()
def width_px(fig: Figure) -> int: return fig.width_px()
def height_px(fig: Figure) -> int: return fig.height_px()
def to_line_triplet(fig: Figure): return fig.to_line_triplet()


def new_figure(width_px: int, height_px: int, title: str = "", y_name: str = "") -> Figure:
    return Figure(title, y_name, width_px, height_px)


def theme_light() -> str: return "light"
def theme_dark() -> str: return "dark"
def theme_vintage() -> str: return "vintage"


def _base(title, trigger="axis"):
    return {"title": {"text": title}, "tooltip": {"trigger": trigger}}


def _xy(x, y_series, names, kind, title, y_name, **per_series):
    opt = _base(title)
    opt["legend"] = {"data": list(names)}
    opt["xAxis"] = {"type": "category", "data": list(x)}
    opt["yAxis"] = {"type": "value", "name": y_name}
    opt["series"] = [dict({"type": kind, "name": names[i] if i < len(names) else f"s{i}", "data": list(ys)}, **per_series)
                     for i, ys in enumerate(y_series)]
    return opt


def echarts_bar_option(x, y_series, series_names, stacked: bool = False, title: str = "Bar Chart",
                       y_name: str = "value") -> str:
    return dumps(_xy(x, y_series, series_names, "bar", title, y_name, **({"stack": "total"} if stacked else {})))


def echarts_line_option(x, y_series, series_names, smooth: bool = True, area: bool = False,
                        title: str = "Line Chart", y_name: str = "value") -> str:
    extra = {"smooth": bool(smooth)}
    if area:
        extra["areaStyle"] = {}
    return dumps(_xy(x, y_series, series_names, "line", title, y_name, **extra))


def echarts_scatter_option(x, y, title: str = "Scatter", x_name: str = "x", y_name: str = "y") -> str:
    opt = _base(title, "item")
    opt.update(xAxis={"type": "value", "name": x_name}, yAxis={"type": "value", "name": y_name},
               series=[{"type": "scatter", "data": [[a, b] for a, b in zip(x, y)]}])
    return dumps(opt)


def echarts_effectscatter_option(points, title: str = "EffectScatter") -> str:
    opt = _base(title, "item")
    opt.update(xAxis={"type": "value"}, yAxis={"type": "value"},
               series=[{"type": "effectScatter", "rippleEffect": {"brushType": "stroke"},
                        "data": [[a, b] for a, b in points]}])
    return dumps(opt)


def _named(labels, values):
    return [{"name": n, "value": v} for n, v in zip(labels, values)]


def echarts_pie_option(labels, values, title: str = "Pie") -> str:
    opt = _base(title, "item")
    opt["series"] = [{"type": "pie", "radius": "60%", "data": _named(labels, values)}]
    return dumps(opt)


def echarts_funnel_option(labels, values, title: str = "Funnel") -> str:
    opt = _base(title, "item")
    opt["series"] = [{"type": "funnel", "data": _named(labels, values)}]
    return dumps(opt)


def echarts_sunburst_option(labels, values, title: str = "Sunburst") -> str:
    opt = _base(title, "item")
    opt["series"] = [{"type": "sunburst", "radius": [0, "90%"], "data": _named(labels, values)}]
    return dumps(opt)


def echarts_treemap_option(names, values, title: str = "Treemap") -> str:
    opt = _base(title, "item")
    opt["series"] = [{"type": "treemap", "data": _named(names, values)}]
    return dumps(opt)


def echarts_gauge_option(value: float, title: str = "Gauge", unit: str = "%") -> str:
    opt = {"title": {"text": title}, "tooltip": {},
           "series": [{"type": "gauge", "detail": {"formatter": "{value}" + unit}, "data": [{"value": value}]}]}
    return dumps(opt)


def echarts_heatmap_option(x_labels, y_labels, values, title: str = "Heatmap") -> str:
    data, flat = [], []
    for yi in range(min(len(y_labels), len(values))):
        for xi in range(min(len(x_labels), len(values[yi]))):
            data.append([xi, yi, values[yi][xi]])
            flat.append(values[yi][xi])
    opt = _base(title, "item")
    opt.update(xAxis={"type": "category", "data": list(x_labels)}, yAxis={"type": "category", "data": list(y_labels)},
               visualMap={"min": min(flat) if flat else 0, "max": max(flat) if flat else 1, "calculable": True,
                          "orient": "horizontal", "left": "center", "bottom": 10},
               series=[{"type": "heatmap", "data": data}])
    return dumps(opt)


def echarts_candlestick_option(x, o, h, l, c, title: str = "Candlestick") -> str:
    opt = _base(title)
    opt.update(xAxis={"type": "category", "data": list(x)}, yAxis={"type": "value", "scale": True},
               series=[{"type": "candlestick", "data": [[a, b, d, e] for a, b, d, e in zip(o, c, l, h)]}])
    return dumps(opt)


def echarts_calendar_option(range_str: str, items, title: str = "Calendar Heatmap") -> str:
    vals = [v for _, v in items]
    opt = _base(title, "item")
    opt.update(calendar={"range": range_str},
               visualMap={"min": min(vals) if vals else 0, "max": max(vals) if vals else 1, "orient": "horizontal",
                          "left": "center", "top": 30},
               series=[{"type": "heatmap", "coordinateSystem": "calendar", "data": [[d, v] for d, v in items]}])
    return dumps(opt)


def echarts_custom_option(raw_option_json: str) -> str:
    return raw_option_json


def echarts_lines_option(lines, title: str = "Geo Lines") -> str:
    opt = _base(title, "item")
    opt.update(geo={"map": "world", "roam": True},
               series=[{"type": "lines", "coordinateSystem": "geo",
                        "data": [{"coords": [[a[0], a[1]], [b[0], b[1]]]} for a, b in lines]}])
    return dumps(opt)


def echarts_map_option(pairs, title: str = "World Map Choropleth") -> str:
    vals = [v for _, v in pairs]
    opt = _base(title, "item")
    opt.update(visualMap={"min": min(vals) if vals else 0, "max": max(vals) if vals else 1, "calculable": True},
               series=[{"type": "map", "map": "world", "roam": True, "data": [{"name": n, "value": v} for n, v in pairs]}])
    return dumps(opt)


def echarts_parallel_option(dim_names, rows, title: str = "Parallel") -> str:
    opt = {"title": {"text": title}, "parallelAxis": [{"dim": i, "name": n} for i, n in enumerate(dim_names)],
           "parallel": {}, "series": [{"type": "parallel", "data": [list(r) for r in rows]}]}
    return dumps(opt)


def echarts_pictorialbar_option(x, values, title: str = "PictorialBar", symbol: str = "rect") -> str:
    opt = _base(title)
    opt.update(xAxis={"type": "category", "data": list(x)}, yAxis={"type": "value"},
               series=[{"type": "pictorialBar", "symbol": symbol, "symbolRepeat": True, "data": list(values)}])
    return dumps(opt)


def echarts_radar_option(indicators, series, series_names, title: str = "Radar") -> str:
    opt = _base(title, "item")
    opt.update(legend={"data": list(series_names)},
               radar={"indicator": [{"name": n, "max": m} for n, m in indicators]},
               series=[{"type": "radar", "data": [{"name": series_names[i] if i < len(series_names) else f"s{i}",
                                                   "value": list(v)} for i, v in enumerate(series)]}])
    return dumps(opt)


def echarts_sankey_option(nodes, links, title: str = "Sankey") -> str:
    opt = _base(title, "item")
    opt["series"] = [{"type": "sankey", "data": [{"name": n} for n in nodes],
                      "links": [{"source": s, "target": t, "value": v} for s, t, v in links]}]
    return dumps(opt)


def echarts_themeriver_option(dates, names, matrix, title: str = "ThemeRiver") -> str:
    data = [[d, matrix[di][ni], names[ni]] for di, d in enumerate(dates) if di < len(matrix)
            for ni in range(min(len(names), len(matrix[di])))]
    opt = _base(title)
    opt.update(singleAxis={"type": "time"}, legend={"data": list(names)}, series=[{"type": "themeRiver", "data": data}])
    return dumps(opt)


def echarts_dashboard_html(options: Sequence[str], titles: Sequence[str], layout: str = "grid") -> str:
    cols = "repeat(auto-fit,minmax(480px,1fr))" if layout == "grid" else "1fr"
    cells, inits = [], []
    for i, opt in enumerate(options):
        t = escape_html(titles[i]) if i < len(titles) else f"Chart {i + 1}"
        cells.append(f"<div class='cell'><h3>{t}</h3><div id='c{i}' style='width:100%;height:400px'></div></div>")
        inits.append(f"echarts.init(document.getElementById('c{i}')).setOption({opt});")
    return ("<!doctype html><html><head><meta charset='utf-8'>"
            "<meta name='viewport' content='width=device-width,initial-scale=1'>"
            f"<script src='{ECHARTS_CDN}'></script>"
            f"<style>body{{font-family:sans-serif;margin:12px}}.grid{{display:grid;grid-template-columns:{cols};gap:12px}}"
            ".cell{border:1px solid #ddd;border-radius:6px;padding:8px}</style></head><body>"
            f"<div class='grid'>{''.join(cells)}</div><script>{''.join(inits)}</script></body></html>")


# ---- numeric helpers ---------------------------------------------------------------------------------------
def hist1d(samples, bins: int, minv: float, maxv: float) -> List[int]:
    out = [0] * max(int(bins), 0)
    if not out or maxv <= minv:
        return out
    w = (maxv - minv) / len(out)
    for s in samples:
        if minv <= s <= maxv:
            out[min(int((s - minv) / w), len(out) - 1)] += 1
    return out


def kde_1d(samples, xs, bandwidth: float) -> List[float]:
    n = len(samples)
    if n == 0 or bandwidth <= 0:
        return [0.0] * len(xs)
    k = 1.0 / (n * bandwidth * math.sqrt(2.0 * math.pi))
    return [k * sum(math.exp(-0.5 * ((x - s) / bandwidth) ** 2) for s in samples) for x in xs]


def marching_squares(grid, level: float):
    """Iso-line segments ``[[x0, y0], [x1, y1]]`` of a row-major grid at ``level`` (cell corners at integers)."""
    segs = []
    H = len(grid)
    W = len(grid[0]) if H else 0

    def interp(a, b, pa, pb):
        t = 0.5 if a == b else (level - a) / (b - a)
        return [pa[0] + t * (pb[0] - pa[0]), pa[1] + t * (pb[1] - pa[1])]

    for y in range(H - 1):
        for x in range(W - 1):
            v = [grid[y][x], grid[y][x + 1], grid[y + 1][x + 1], grid[y + 1][x]]
            p = [(x, y), (x + 1, y), (x + 1, y + 1), (x, y + 1)]
            idx = sum(1 << i for i in range(4) if v[i] >= level)
            if idx in (0, 15):
                continue
            edge = lambda i: interp(v[i], v[(i + 1) % 4], p[i], p[(i + 1) % 4])
            table = {1: [(3, 0)], 2: [(0, 1)], 3: [(3, 1)], 4: [(1, 2)], 5: [(3, 0), (1, 2)], 6: [(0, 2)], 7: [(3, 2)],
                     8: [(2, 3)], 9: [(0, 2)], 10: [(0, 1), (2, 3)], 11: [(1, 2)], 12: [(1, 3)], 13: [(0, 1)],
                     14: [(3, 0)]}
            for a, b in table[idx]:
                segs.append([edge(a), edge(b)])
    return segs


# ---- exporters -----------------------------------------------------------------------------------------------
@dataclass
class EChartsConfig:
    theme: str = ""
    include_gl: bool = False
    width_px: int = 960
    height_px: int = 540


class ChartExporter:
    """``name`` plus ``export_html(fig, path)``; looked up by flavour."""

    def __init__(self, name: str, fn: Callable[[Figure, str], bool]):
        self._name, self._fn = name, fn

    def name(self) -> str:
        return self._name

    def export_html(self, fig: Figure, path: str) -> bool:
        return self._fn(fig, path)


class EChartsExporter(ChartExporter):
    def __init__(self, config: EChartsConfig = None):
        self.config = config or EChartsConfig()
        super().__init__("echarts", self._export)

    def _export(self, fig: Figure, path: str) -> bool:
        xs, ys, names = fig.to_line_triplet()
        opt = echarts_line_option(xs, ys, names, title=fig.title(), y_name=fig.y_label())
        return write_text(path, echarts_html(opt, fig.title() or "Chart", fig.width_px(), fig.height_px(),
                                             theme=self.config.theme, include_gl=self.config.include_gl))


def make_echarts_exporter() -> Optional[ChartExporter]:
    return EChartsExporter()


def get_exporter(flavor: str) -> Optional[ChartExporter]:
    return make_echarts_exporter() if flavor.lower() == "echarts" else None


def name(exporter: ChartExporter) -> str:
    return exporter.name()


def export_html(exporter: ChartExporter, fig: Figure, path: str) -> bool:
    return exporter.export_html(fig, path)


def export_figure_html(fig: Figure, path: str, flavor: str = "echarts", auto_open: bool = False) -> bool:
    ex = get_exporter(flavor)
    if ex is None:
        print("exporter not available: " + flavor)
        return False
    return ex.export_html(fig, path)
