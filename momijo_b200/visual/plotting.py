"""``chart_*`` option builders and axis / layout fragments (legacy/src/momijo/visual/plotting/
echarts_series.mojo, echarts_custom.mojo, echarts_3d.mojo, echarts_polar.mojo, echarts_sankey.mojo,
echarts_axes.mojo, echarts_layout.mojo, boxplot.mojo, graph.mojo, violin_utils.mojo). Each returns an
ECharts option (or fragment) as a JSON string."""
from __future__ import annotations

import math
from typing import List, Sequence, Tuple

from .core import dumps, json_string_array


# ---- axes / layout fragments -------------------------------------------------------------------------------
def axis_value() -> str: return dumps({"type": "value"})
def axis_log(base: int = 10) -> str: return dumps({"type": "log", "logBase": int(base)})
def axis_time() -> str: return dumps({"type": "time"})
def axis_category(labels: Sequence[str]) -> str: return dumps({"type": "category", "data": list(labels)})
def angle_axis_category(labels: Sequence[str]) -> str: return dumps({"type": "category", "data": list(labels)})
def radius_axis_value() -> str: return dumps({"type": "value"})


def parallel_axis(dim: int, name: str, axis_type: str = "value") -> str:
    return dumps({"dim": int(dim), "name": name, "type": axis_type})


def visualMap_continuous(minv: float, maxv: float, orient: str = "horizontal") -> str:
    return dumps({"type": "continuous", "min": minv, "max": maxv, "calculable": True, "orient": orient,
                  "left": "center", "bottom": 10})


def visualMap_piecewise(pieces, orient: str = "horizontal") -> str:
    from .core import loads
    p = loads(pieces) if isinstance(pieces, str) else pieces
    return dumps({"type": "piecewise", "pieces": p, "orient": orient, "left": "center", "bottom": 10})


def timeline_builder(labels: Sequence[str]) -> str:
    return dumps({"axisType": "category", "autoPlay": False, "data": list(labels)})


def dataset_builder(source) -> str:
    from .core import loads
    return dumps({"source": loads(source) if isinstance(source, str) else source})


def _wrap(title, series, x_axis=None, y_axis=None, trigger="axis", **extra):
    opt = {"title": {"text": title}, "tooltip": {"trigger": trigger}}
    if x_axis is not None:
        opt["xAxis"] = x_axis
    if y_axis is not None:
        opt["yAxis"] = y_axis
    opt.update(extra)
    opt["series"] = series if isinstance(series, list) else [series]
    return dumps(opt)


_V = {"type": "value"}


# ---- cartesian series --------------------------------------------------------------------------------------
def chart_line(title, xs, ys, step: bool = False, area: bool = False) -> str:
    s = {"type": "line", "data": [[x, y] for x, y in zip(xs, ys)], "showSymbol": False}
    if step:
        s["step"] = "middle"
    if area:
        s["areaStyle"] = {}
    return _wrap(title, s, _V, _V)


def chart_bar(title, labels, values, horizontal: bool = False, stacked_key: str = "") -> str:
    s = {"type": "bar", "data": list(values)}
    if stacked_key:
        s["stack"] = stacked_key
    cat = {"type": "category", "data": list(labels)}
    return _wrap(title, s, _V if horizontal else cat, cat if horizontal else _V)


def chart_scatter(title, xs, ys, sizes=None) -> str:
    sizes = list(sizes or [])
    data = [[x, y] + ([sizes[i]] if i < len(sizes) else []) for i, (x, y) in enumerate(zip(xs, ys))]
    s = {"type": "scatter", "data": data}
    if sizes:
        s["symbolSize"] = "__fn__size"
    out = _wrap(title, s, _V, _V, trigger="item")
    return out.replace('"__fn__size"', "function(d){return d[2];}")


def chart_pie(title, labels, values, donut: bool = False) -> str:
    s = {"type": "pie", "radius": ["40%", "70%"] if donut else "60%",
         "data": [{"name": n, "value": v} for n, v in zip(labels, values)]}
    return _wrap(title, s, trigger="item")


def chart_heatmap(title, rows: int, cols: int, values) -> str:
    vals = list(values)
    data = [[c, r, vals[r * cols + c]] for r in range(rows) for c in range(cols) if r * cols + c < len(vals)]
    lo, hi = (min(vals), max(vals)) if vals else (0, 1)
    return _wrap(title, {"type": "heatmap", "data": data},
                 {"type": "category", "data": list(range(cols))}, {"type": "category", "data": list(range(rows))},
                 trigger="item", visualMap={"min": lo, "max": hi, "calculable": True, "orient": "horizontal",
                                            "left": "center", "bottom": 10})


def _percentile(sorted_vals, p: float) -> float:
    if not sorted_vals:
        return 0.0
    pos = (len(sorted_vals) - 1) * p
    lo, hi = int(math.floor(pos)), int(math.ceil(pos))
    return sorted_vals[lo] + (sorted_vals[hi] - sorted_vals[lo]) * (pos - lo)


def five_number(values) -> List[float]:
    s = sorted(float(v) for v in values)
    return [s[0], _percentile(s, 0.25), _percentile(s, 0.5), _percentile(s, 0.75), s[-1]] if s else [0.0] * 5


def chart_boxplot(title, groups) -> str:
    return _wrap(title, {"type": "boxplot", "data": [five_number(g) for g in groups]},
                 {"type": "category", "data": [str(i + 1) for i in range(len(groups))]}, _V, trigger="item")


def echarts_boxplot_option(x_labels, values, title: str = "Boxplot") -> str:
    return _wrap(title, {"type": "boxplot", "data": [five_number(g) for g in values]},
                 {"type": "category", "data": list(x_labels)}, _V, trigger="item")


def echarts_graph_option(nodes, links: Sequence[Tuple[int, int]], title: str = "Graph") -> str:
    names = list(nodes)
    s = {"type": "graph", "layout": "force", "roam": True, "label": {"show": True},
         "data": [{"name": n} for n in names],
         "links": [{"source": names[a], "target": names[b]} for a, b in links if a < len(names) and b < len(names)]}
    return _wrap(title, s, trigger="item")


# ---- custom-series charts ----------------------------------------------------------------------------------
def chart_stem(title, xs, ys, baseline: float = 0.0) -> str:
    stems = {"type": "custom", "renderItem": "__fn__stem", "data": [[x, y] for x, y in zip(xs, ys)]}
    heads = {"type": "scatter", "data": [[x, y] for x, y in zip(xs, ys)]}
    out = _wrap(title, [stems, heads], _V, _V)
    fn = ("function(p,api){var a=api.coord([api.value(0),%s]),b=api.coord([api.value(0),api.value(1)]);"
          "return {type:'line',shape:{x1:a[0],y1:a[1],x2:b[0],y2:b[1]},style:{stroke:api.visual('color')}};}" % repr(float(baseline)))
    return out.replace('"__fn__stem"', fn)


def chart_errorbar(title, xs, ys, yerr) -> str:
    bars = {"type": "custom", "renderItem": "__fn__err", "data": [[x, y - e, y + e] for x, y, e in zip(xs, ys, yerr)]}
    pts = {"type": "scatter", "data": [[x, y] for x, y in zip(xs, ys)]}
    out = _wrap(title, [bars, pts], _V, _V)
    fn = ("function(p,api){var a=api.coord([api.value(0),api.value(1)]),b=api.coord([api.value(0),api.value(2)]);"
          "return {type:'group',children:[{type:'line',shape:{x1:a[0],y1:a[1],x2:b[0],y2:b[1]},style:{stroke:'#333'}},"
          "{type:'line',shape:{x1:a[0]-4,y1:a[1],x2:a[0]+4,y2:a[1]},style:{stroke:'#333'}},"
          "{type:'line',shape:{x1:b[0]-4,y1:b[1],x2:b[0]+4,y2:b[1]},style:{stroke:'#333'}}]};}")
    return out.replace('"__fn__err"', fn)


def _ints(n: int) -> List[int]:
    return list(range(n))


def _violin_curve(samples, points: int = 40):
    s = sorted(float(v) for v in samples)
    if len(s) < 2:
        return [], []
    lo, hi = s[0], s[-1]
    n = len(s)
    mean = sum(s) / n
    sd = math.sqrt(sum((v - mean) ** 2 for v in s) / max(n - 1, 1)) or 1.0
    bw = 1.06 * sd * n ** (-0.2)
    grid = [lo + (hi - lo) * i / (points - 1) for i in range(points)]
    dens = [sum(math.exp(-0.5 * ((g - v) / bw) ** 2) for v in s) / (n * bw * math.sqrt(2 * math.pi)) for g in grid]
    return grid, dens


def _compute_violin_curve_json(samples, points: int = 40) -> str:
    g, d = _violin_curve(samples, points)
    return dumps([[a, b] for a, b in zip(g, d)])


def chart_violin(title, categories, xs, ys) -> str:
    """``xs[i]`` are density values and ``ys[i]`` the positions of category ``i`` (a mirrored outline)."""
    series = []
    for i, name in enumerate(categories):
        dens, pos = list(xs[i]), list(ys[i])
        peak = max(dens) if dens else 1.0
        half = [(0.4 * d / (peak or 1.0)) for d in dens]
        outline = [[i + h, p] for h, p in zip(half, pos)] + [[i - h, p] for h, p in reversed(list(zip(half, pos)))]
        series.append({"type": "line", "name": name, "data": outline, "showSymbol": False, "areaStyle": {"opacity": 0.4},
                       "lineStyle": {"width": 1}})
    return _wrap(title, series, {"type": "value", "min": -0.5, "max": len(categories) - 0.5}, _V, trigger="item")


def chart_eventplot(title, rows: int, events) -> str:
    data = [[t, r] for r in range(min(rows, len(events))) for t in events[r]]
    s = {"type": "scatter", "symbol": "rect", "symbolSize": [2, 18], "data": data}
    return _wrap(title, s, _V, {"type": "category", "data": list(range(rows))}, trigger="item")


def chart_contour_lines(title, lines) -> str:
    series = [{"type": "line", "data": [[p[0], p[1]] for p in ln], "showSymbol": False} for ln in lines]
    return _wrap(title, series, _V, _V, trigger="item")


def chart_hexbin(title, centers, size: float, values, vmin: float, vmax: float) -> str:
    data = [[c[0], c[1], v] for c, v in zip(centers, values)]
    s = {"type": "scatter", "symbol": "path://M0,-1L0.866,-0.5L0.866,0.5L0,1L-0.866,0.5L-0.866,-0.5Z",
         "symbolSize": size, "data": data}
    return _wrap(title, s, _V, _V, trigger="item",
                 visualMap={"min": vmin, "max": vmax, "dimension": 2, "calculable": True})


def chart_quiver(title, xs, ys, u, v, scale: float = 1.0) -> str:
    data = [[x, y, x + a * scale, y + b * scale] for x, y, a, b in zip(xs, ys, u, v)]
    out = _wrap(title, {"type": "custom", "renderItem": "__fn__quiver", "data": data}, _V, _V, trigger="item")
    fn = ("function(p,api){var a=api.coord([api.value(0),api.value(1)]),b=api.coord([api.value(2),api.value(3)]);"
          "var t=Math.atan2(b[1]-a[1],b[0]-a[0]),h=6;return {type:'group',children:["
          "{type:'line',shape:{x1:a[0],y1:a[1],x2:b[0],y2:b[1]},style:{stroke:'#1f77b4'}},"
          "{type:'polygon',shape:{points:[[b[0],b[1]],[b[0]-h*Math.cos(t-0.4),b[1]-h*Math.sin(t-0.4)],"
          "[b[0]-h*Math.cos(t+0.4),b[1]-h*Math.sin(t+0.4)]]},style:{fill:'#1f77b4'}}]};}")
    return out.replace('"__fn__quiver"', fn)


# ---- polar / sankey ----------------------------------------------------------------------------------------
def _polar(title, kind, theta, r, **extra) -> str:
    s = {"type": kind, "coordinateSystem": "polar", "data": [[rr, t] for t, rr in zip(theta, r)]}
    s.update(extra)
    return dumps({"title": {"text": title}, "tooltip": {"trigger": "item"}, "polar": {},
                  "angleAxis": {"type": "value", "min": 0, "max": 360}, "radiusAxis": {"type": "value"}, "series": [s]})


def chart_polar_line(title, theta, r) -> str: return _polar(title, "line", theta, r, showSymbol=False)
def chart_polar_scatter(title, theta, r) -> str: return _polar(title, "scatter", theta, r)
def chart_polar_bar(title, theta, r) -> str: return _polar(title, "bar", theta, r)


def chart_sankey(title, nodes, links) -> str:
    ls = [{"source": l[0], "target": l[1], "value": float(l[2]) if len(l) > 2 else 1.0} for l in links]
    return _wrap(title, {"type": "sankey", "data": [{"name": n} for n in nodes], "links": ls}, trigger="item")


# ---- 3-D (echarts-gl) ----------------------------------------------------------------------------------------
def _wrap3d(title, series) -> str:
    return dumps({"title": {"text": title}, "tooltip": {}, "xAxis3D": {"type": "value"}, "yAxis3D": {"type": "value"},
                  "zAxis3D": {"type": "value"}, "grid3D": {}, "series": series if isinstance(series, list) else [series]})


def chart_surface3d(title, rows: int, cols: int, zvals) -> str:
    z = list(zvals)
    data = [[c, r, z[r * cols + c]] for r in range(rows) for c in range(cols) if r * cols + c < len(z)]
    return _wrap3d(title, {"type": "surface", "data": data, "dataShape": [rows, cols]})


def chart_line3d(title, path) -> str: return _wrap3d(title, {"type": "line3D", "data": [list(p) for p in path]})
def chart_scatter3d(title, points) -> str: return _wrap3d(title, {"type": "scatter3D", "data": [list(p) for p in points]})
def chart_bar3d(title, bars) -> str: return _wrap3d(title, {"type": "bar3D", "data": [list(p) for p in bars]})


def chart_lines3d(title, segments) -> str:
    return _wrap3d(title, {"type": "lines3D", "coordinateSystem": "cartesian3D",
                           "data": [[list(p) for p in seg] for seg in segments]})


def chart_globe_with_textures(title, baseTextureUrl: str, heightTextureUrl: str) -> str:
    return dumps({"title": {"text": title}, "globe": {"baseTexture": baseTextureUrl, "heightTexture": heightTextureUrl,
                                                      "shading": "lambert", "viewControl": {"autoRotate": True}},
                  "series": []})


def chart_geo3d_world(title, map_name: str, geojson_url: str) -> str:
    return dumps({"title": {"text": title}, "geo3D": {"map": map_name, "shading": "lambert"}, "series": [],
                  "__geojson_url": geojson_url})
