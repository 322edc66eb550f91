"""Option assemblers: ``Option`` takes pre-serialised JSON fragments per top-level key
(legacy/src/momijo/visual/charts/option.mojo:67-375); ``EasyOption`` builds the fragments from plain
arguments (legacy/src/momijo/visual/charts/ez_option.mojo:100-2200). Both end in ``to_json()``."""
from __future__ import annotations

from typing import Dict, List, Sequence

from .core import dumps, loads
from .plotting import five_number


def series_bar(name: str, data: Sequence[int]) -> str:
    return dumps({"type": "bar", "name": name, "data": list(data)})


def series_line(name: str, data: Sequence[int]) -> str:
    return dumps({"type": "line", "name": name, "data": list(data)})


def _frag(x):
    """Accept a JSON string or an already-built object."""
    return loads(x) if isinstance(x, str) else x


class Option:
    _single = {"title": "title", "tooltip": "tooltip", "legend": "legend", "grid": "grid", "toolbox": "toolbox",
               "visual_map": "visualMap", "timeline": "timeline", "calendar": "calendar", "graphic": "graphic",
               "aria": "aria", "axis_pointer": "axisPointer", "dataset": "dataset", "geo": "geo", "parallel": "parallel",
               "xaxis_json": "xAxis", "yaxis_json": "yAxis", "single_axis": "singleAxis", "polar": "polar",
               "radar": "radar", "angle_axis": "angleAxis", "radius_axis": "radiusAxis", "xaxis3d_json": "xAxis3D",
               "yaxis3d_json": "yAxis3D", "zaxis3d_json": "zAxis3D", "grid3d_json": "grid3D"}

    def __init__(self):
        self._d: Dict[str, object] = {}
        self._series: List[object] = []
        self._datazoom: List[object] = []
        self._parallel_axis: List[object] = []
        self._colors: List[str] = []

    def set_subtitle(self, text: str, subtext: str):
        self._d["title"] = {"text": text, "subtext": subtext}
        return self

    def set_background(self, color: str):
        self._d["backgroundColor"] = color
        return self

    def set_parallel_axis(self, json_obj):
        v = _frag(json_obj)
        self._parallel_axis.extend(v if isinstance(v, list) else [v])
        return self

    def set_xaxis_category(self, categories: Sequence[str]):
        self._d["xAxis"] = {"type": "category", "data": list(categories)}
        return self

    def set_yaxis_value(self):
        self._d["yAxis"] = {"type": "value"}
        return self

    def set_colors(self, colors: Sequence[str]):
        self._colors = list(colors)
        return self

    def add_color(self, color: str):
        self._colors.append(color)
        return self

    def add_series_json(self, s_json):
        self._series.append(_frag(s_json))
        return self

    def add_datazoom_json(self, dz_json):
        self._datazoom.append(_frag(dz_json))
        return self

    def set_animation(self, enabled: bool, duration: int = 1000, easing: str = "cubicOut"):
        self._d.update(animation=bool(enabled), animationDuration=int(duration), animationEasing=easing)
        return self

    def to_dict(self) -> dict:
        out = dict(self._d)
        if self._colors:
            out["color"] = list(self._colors)
        if self._parallel_axis:
            out["parallelAxis"] = list(self._parallel_axis)
        if self._datazoom:
            out["dataZoom"] = list(self._datazoom)
        out["series"] = list(self._series)
        return out

    def to_json(self) -> str:
        return dumps(self.to_dict())



def _make_fragment_setter(key: str):
    def setter(self, fragment):
        self._d[key] = _frag(fragment)
        return self
    setter.__doc__ = f"Set the ``{key}`` component from a JSON fragment (string or object)."
    return setter


for _short, _key in Option._single.items():
    setattr(Option, "set_" + _short, _make_fragment_setter(_key))

class EasyOption:
    """Fluent builder; every ``add_*`` appends a series, every ``set_*`` fills a top-level component."""

    def __init__(self):
        self.o: Dict[str, object] = {}
        self.series: List[dict] = []
        self.titles: List[dict] = []
        self.datazoom: List[dict] = []
        self.parallel_axes: List[dict] = []
        self.extra: List[str] = []

    # ---- look ----
    def set_color(self, colors):
        self.o["color"] = list(colors); return self

    def set_background(self, css_color):
        self.o["backgroundColor"] = css_color; return self

    def add_title(self, text, left="center", top=10, font_size=18, color="#333", subtext=""):
        t = {"text": text, "left": left, "top": top, "textStyle": {"fontSize": font_size, "color": color}}
        if subtext:
            t["subtext"] = subtext
        self.titles.append(t); return self

    def set_title(self, text, left="center", top=10, font_size=18, color="#333", subtext=""):
        self.titles = []
        return self.add_title(text, left, top, font_size, color, subtext)

    def _tooltip(self, trigger, pointer=None, bg="#fff", border="#aaa", text_color="#333", formatter=None):
        t = {"trigger": trigger, "backgroundColor": bg, "borderColor": border, "textStyle": {"color": text_color}}
        if pointer:
            t["axisPointer"] = {"type": pointer}
        if formatter:
            t["formatter"] = formatter
        self.o["tooltip"] = t; return self

    def set_tooltip_axis_shadow(self, bg="#fff", border="#aaa", text_color="#333"):
        return self._tooltip("axis", "shadow", bg, border, text_color)

    def set_tooltip_axis_line(self, bg="#fff", border="#aaa", text_color="#333"):
        return self._tooltip("axis", "line", bg, border, text_color)

    def set_tooltip_axis_cross(self, bg="#fff", border="#aaa", text_color="#333"):
        return self._tooltip("axis", "cross", bg, border, text_color)

    def set_tooltip_item(self, bg="#fff", border="#aaa", text_color="#333", formatter=None):
        return self._tooltip("item", None, bg, border, text_color, formatter)

    set_tooltip_boxplot_item = set_tooltip_item
    set_tooltip_polar_item = set_tooltip_item
    set_tooltip_item_for_radar = set_tooltip_item
    set_tooltip_sunburst = set_tooltip_item

    def set_legend(self, names, top_px=80, font_size=12, color="#333"):
        self.o["legend"] = {"data": list(names), "top": top_px, "textStyle": {"fontSize": font_size, "color": color}}
        return self

    def set_toolbox_default(self, right_px=20, top_px=80, show=True):
        self.o["toolbox"] = {"show": bool(show), "right": right_px, "top": top_px,
                             "feature": {"saveAsImage": {}, "dataView": {"readOnly": True}, "restore": {}}}
        return self

    def set_grid(self, top_px, left_pct, right_pct, bottom_pct, contain_label=True):
        self.o["grid"] = {"top": top_px, "left": left_pct, "right": right_pct, "bottom": bottom_pct,
                          "containLabel": bool(contain_label)}
        return self

    def set_xaxis_category_json(self, name, name_location, name_gap, categories, labels_color="#333", rotate=0):
        self.o["xAxis"] = {"type": "category", "name": name, "nameLocation": name_location, "nameGap": name_gap,
                           "data": list(categories), "axisLabel": {"color": labels_color, "rotate": rotate}}
        return self

    def set_yaxis_value_json(self, name, name_location, name_gap, labels_color="#333"):
        self.o["yAxis"] = {"type": "value", "name": name, "nameLocation": name_location, "nameGap": name_gap,
                           "axisLabel": {"color": labels_color}}
        return self

    def set_xaxis_value(self, name=""):
        self.o["xAxis"] = {"type": "value", "name": name}; return self

    # ---- axis builders of the reference (legacy/src/momijo/visual/charts/ez_option.mojo:2237-2302); ``minv`` / ``maxv``
    # are JSON fragments ("0", "'dataMax'") or numbers ---------------------------------------------------------------
    @staticmethod
    def _value_axis(name, name_location, name_gap, labels_color, minv, maxv):
        ax = {"type": "value", "name": name, "nameLocation": name_location, "nameGap": name_gap,
              "axisLabel": {"color": labels_color}}
        for key, v in (("min", minv), ("max", maxv)):
            if v not in ("", None):
                ax[key] = _frag(v) if isinstance(v, str) else v
        return ax

    def set_xaxis_value_json(self, name, name_location, name_gap, labels_color="#333", minv="", maxv=""):
        self.o["xAxis"] = self._value_axis(name, name_location, name_gap, labels_color, minv, maxv); return self

    def set_yaxis_value_json2(self, name, name_location, name_gap, labels_color="#333", minv="", maxv=""):
        self.o["yAxis"] = self._value_axis(name, name_location, name_gap, labels_color, minv, maxv); return self

    def set_yaxis_category_json(self, name, name_location, name_gap, labels_color, data):
        self.o["yAxis"] = {"type": "category", "name": name, "nameLocation": name_location, "nameGap": name_gap,
                           "axisLabel": {"color": labels_color}, "data": list(data)}
        return self

    @staticmethod
    def _category_axis(labels, name, name_location, name_gap, labels_color, rotate_deg):
        ax = {"type": "category"}
        if name:
            ax.update(name=name, nameLocation=name_location, nameGap=name_gap)
        ax.update(data=list(labels), axisLabel={"color": labels_color, "rotate": rotate_deg})
        return ax

    def set_xaxis_category_labels(self, labels, name="", name_location="middle", name_gap=28, labels_color="#333",
                                  rotate_deg=0):
        self.o["xAxis"] = self._category_axis(labels, name, name_location, name_gap, labels_color, rotate_deg); return self

    def set_yaxis_category_labels(self, labels, name="", name_location="middle", name_gap=28, labels_color="#333",
                                  rotate_deg=0):
        self.o["yAxis"] = self._category_axis(labels, name, name_location, name_gap, labels_color, rotate_deg); return self

    def add_datazoom_slider(self, start_pct=0, end_pct=100):
        self.datazoom.append({"type": "slider", "start": start_pct, "end": end_pct}); return self

    def add_datazoom_inside(self):
        self.datazoom.append({"type": "inside"}); return self

    def set_visualmap(self, minv, maxv, dimension, inrange_colors):
        self.o["visualMap"] = {"min": minv, "max": maxv, "dimension": dimension, "inRange": {"color": list(inrange_colors)}}
        return self

    def set_visualmap_continuous(self, minv, maxv, colors, dimension=2):
        self.o["visualMap"] = {"type": "continuous", "min": minv, "max": maxv, "dimension": dimension, "calculable": True,
                               "inRange": {"color": list(colors)}}
        return self

    def set_animation(self, enabled, duration_ms=1000, easing="cubicOut", delay_per_index_ms=50):
        self.o.update(animation=bool(enabled), animationDuration=duration_ms, animationEasing=easing,
                      animationDelayUpdate=delay_per_index_ms)
        return self

    def add_extra_kv(self, kv_fragment: str):
        """Raw ``"key": value`` text merged into the top level at ``to_json`` time."""
        self.extra.append(kv_fragment); return self

    # ---- cartesian series ----
    def _add(self, kind, name, data, **kw):
        s = {"type": kind, "name": name, "data": data}
        s.update({k: v for k, v in kw.items() if v is not None})
        self.series.append(s); return self

    def add_bar_series(self, name, data, color=None, stack=None, bar_width=None, label_show=False):
        return self._add("bar", name, list(data), itemStyle={"color": color} if color else None, stack=stack,
                         barWidth=bar_width, label={"show": True, "position": "top"} if label_show else None)

    def add_line_series(self, name, data, color=None, smooth=False, symbol="circle", symbol_size=6, width=2, area=False):
        return self._add("line", name, list(data), smooth=bool(smooth), symbol=symbol, symbolSize=symbol_size,
                         lineStyle={"width": width, **({"color": color} if color else {})},
                         itemStyle={"color": color} if color else None, areaStyle={} if area else None)

    def add_area_series(self, name, data, color=None, opacity=0.4, smooth=True, stack=None):
        return self._add("line", name, list(data), smooth=bool(smooth), stack=stack,
                         areaStyle={"opacity": opacity, **({"color": color} if color else {})})

    def add_step_line_series(self, name, data, step="middle", color=None):
        return self._add("line", name, list(data), step=step, itemStyle={"color": color} if color else None)

    def add_scatter_series(self, name, points, color=None, symbol_size=10):
        return self._add("scatter", name, [list(p) for p in points], symbolSize=symbol_size,
                         itemStyle={"color": color} if color else None)

    def add_effect_scatter_series(self, name, points, color=None, symbol_size=12, ripple_scale=3.0):
        return self._add("effectScatter", name, [list(p) for p in points], symbolSize=symbol_size,
                         rippleEffect={"brushType": "stroke", "scale": ripple_scale},
                         itemStyle={"color": color} if color else None)

    def add_pictorial_bar_series(self, name, data, symbol="rect", repeat=True, symbol_size=None, color=None):
        return self._add("pictorialBar", name, list(data), symbol=symbol, symbolRepeat=bool(repeat),
                         symbolSize=symbol_size, itemStyle={"color": color} if color else None)

    def add_waterfall_series(self, name, deltas, up_color="#e15759", down_color="#59a14f"):
        base, up, down, run = [], [], [], 0
        for d in deltas:
            if d >= 0:
                base.append(run); up.append(d); down.append("-")
            else:
                base.append(run + d); up.append("-"); down.append(-d)
            run += d
        self._add("bar", name + "_base", base, stack=name, itemStyle={"color": "transparent"}, silent=True)
        self._add("bar", name + " +", up, stack=name, itemStyle={"color": up_color})
        return self._add("bar", name + " -", down, stack=name, itemStyle={"color": down_color})

    def add_pie_series(self, name, labels, values, radius="60%", center=("50%", "55%"), rose=False, label_show=True):
        return self._add("pie", name, [{"name": n, "value": v} for n, v in zip(labels, values)], radius=radius,
                         center=list(center), roseType="radius" if rose else None, label={"show": bool(label_show)})

    def add_heatmap_series_from_triplets(self, name, triplets, label_show=False):
        return self._add("heatmap", name, [list(t) for t in triplets], label={"show": bool(label_show)})

    # ---- grid fields, distributions and flow lines (ez_option.mojo:2306-2610) -----------------------------------------
    def add_heatmap_series(self, name, xs, ys, z, blur_size: int = 0):
        """Heatmap cells ``[x, y, z[row][col]]`` of a regular grid, rows following ``ys``."""
        data = [[xs[c], ys[r], z[r][c]] for r in range(len(ys)) for c in range(len(xs))]
        return self._add("heatmap", name, data, blurSize=blur_size if blur_size > 0 else None, progressive=0)

    def add_contour_lines(self, name_prefix, xs, ys, z, levels, color="#000000", line_width=1, opacity=100):
        """One line series per level, traced by marching squares over the grid cells. Each crossing cell gives one
        segment (the two saddle cases take one diagonal choice); segments are separated by nulls."""
        H, W = len(ys), len(xs)
        if H < 2 or W < 2:
            return self

        def lerp(a, b, za, zb, lvl):
            return a if zb == za else a + (b - a) * (lvl - za) / (zb - za)

        pairs = {1: (3, 0), 14: (3, 0), 2: (0, 1), 13: (0, 1), 3: (3, 1), 12: (3, 1), 4: (2, 3), 11: (2, 3), 5: (2, 0),
                 6: (2, 1), 9: (2, 1), 7: (2, 1), 8: (2, 1), 10: (3, 1)}
        for lvl in levels:
            data = []
            for r in range(H - 1):
                for c in range(W - 1):
                    xL, xR, yB, yT = xs[c], xs[c + 1], ys[r], ys[r + 1]
                    z00, z10, z01, z11 = z[r][c], z[r][c + 1], z[r + 1][c], z[r + 1][c + 1]
                    idx = (z00 > lvl) + 2 * (z10 > lvl) + 4 * (z01 > lvl) + 8 * (z11 > lvl)
                    if idx in (0, 15):
                        continue
                    edge = {0: (lerp(xL, xR, z00, z10, lvl), yB), 1: (xR, lerp(yB, yT, z10, z11, lvl)),
                            2: (lerp(xL, xR, z01, z11, lvl), yT), 3: (xL, lerp(yB, yT, z00, z01, lvl))}
                    a, b = (edge[e] for e in pairs[idx])
                    data += [[a[0], a[1]], [b[0], b[1]], None]
            self._add("line", f"{name_prefix} {lvl}", data, symbol="none",
                      lineStyle={"width": line_width, "color": color, "opacity": opacity / 100})
        return self

    def add_ecdf_series(self, name, samples, color, survival=False, normalized=True, step_style="end",
                        show_symbol=False, line_width=2, area_opacity=0, show_labels=False, label_fmt="{c}"):
        """Empirical CDF (or survival ``1 - F``) of integer samples as a step line: one point per distinct value, the
        probability truncated to six decimals like the reference's integer arithmetic; counts when not normalised."""
        xs = sorted(int(v) for v in samples)
        n = len(xs)
        data, cum, i = [], 0, 0
        while i < n:
            run = 1
            while i + run < n and xs[i + run] == xs[i]:
                run += 1
            cum += run
            if normalized:
                scaled = (cum * 1_000_000) // n
                y = (min(max(1_000_000 - scaled, 0), 1_000_000) if survival else scaled) / 1_000_000
            else:
                y = n - cum if survival else cum
            data.append([xs[i], y])
            i += run
        kw = dict(step=step_style, lineStyle={"width": line_width}, itemStyle={"color": color})
        if not show_symbol or n == 0:
            kw["showSymbol"] = False
        if area_opacity > 0:
            kw["areaStyle"] = {"opacity": area_opacity / 100}
        if show_labels:
            kw["label"] = {"show": True, "position": "top", "formatter": label_fmt}
        return self._add("line", name, data if n else [[0, 0]], **kw)

    def add_survival_series(self, name, samples, color, normalized=True, step_style="end", show_symbol=False,
                            line_width=2, area_opacity=0, show_labels=False, label_fmt="{c}"):
        return self.add_ecdf_series(name, samples, color, True, normalized, step_style, show_symbol, line_width,
                                    area_opacity, show_labels, label_fmt)

    def add_streamlines_series(self, name, polylines_x, polylines_y, color="#5470C6", width=1, opacity=85,
                               show_effect=True, effect_speed=20, effect_size=2, trail_length=30):
        """Polylines on the cartesian grid (``lines`` series), optionally with the moving-dot effect; lines with fewer
        than two points or mismatched coordinate lists are skipped."""
        data = [{"coords": [[x, y] for x, y in zip(px, py)]} for px, py in zip(polylines_x, polylines_y)
                if len(px) > 1 and len(px) == len(py)]
        effect = {"show": True, "constantSpeed": effect_speed, "trailLength": trail_length / 100,
                  "symbolSize": effect_size} if show_effect else None
        return self._add("lines", name, data, coordinateSystem="cartesian2d", polyline=True,
                         lineStyle={"color": color, "width": width, "opacity": opacity / 100}, effect=effect)

    def add_boxplot_series_from_fivenum(self, name, fivenums, color=None):
        return self._add("boxplot", name, [list(f) for f in fivenums], itemStyle={"borderColor": color} if color else None)

    def add_boxplot_series_from_samples(self, name, groups, color=None):
        return self.add_boxplot_series_from_fivenum(name, [five_number(g) for g in groups], color)

    def add_boxplot_outliers(self, name, points, color="#d62728", symbol_size=6):
        return self._add("scatter", name, [list(p) for p in points], symbolSize=symbol_size, itemStyle={"color": color})

    def add_candlestick_series(self, name, ohlc, up_color="#ec0000", down_color="#00da3c"):
        return self._add("candlestick", name, [[o, c, l, h] for o, h, l, c in ohlc],
                         itemStyle={"color": up_color, "color0": down_color, "borderColor": up_color,
                                    "borderColor0": down_color})

    def _custom(self, name, data, js, **kw):
        s = {"type": "custom", "name": name, "data": data, "renderItem": "@@" + js + "@@"}
        s.update(kw)
        self.series.append(s); return self

    def add_stem_series(self, name, xs, ys, baseline=0.0, color="#1f77b4", symbol_size=8):
        js = ("function(p,api){var a=api.coord([api.value(0),%r]),b=api.coord([api.value(0),api.value(1)]);"
              "return {type:'line',shape:{x1:a[0],y1:a[1],x2:b[0],y2:b[1]},style:{stroke:'%s'}};}" % (float(baseline), color))
        self._custom(name + "_stems", [[x, y] for x, y in zip(xs, ys)], js)
        return self.add_scatter_series(name, list(zip(xs, ys)), color, symbol_size)

    def add_errorbar_series(self, name, xs, lows, highs, color="#333", cap=4):
        js = ("function(p,api){var a=api.coord([api.value(0),api.value(1)]),b=api.coord([api.value(0),api.value(2)]),c=%d;"
              "return {type:'group',children:[{type:'line',shape:{x1:a[0],y1:a[1],x2:b[0],y2:b[1]},style:{stroke:'%s'}},"
              "{type:'line',shape:{x1:a[0]-c,y1:a[1],x2:a[0]+c,y2:a[1]},style:{stroke:'%s'}},"
              "{type:'line',shape:{x1:b[0]-c,y1:b[1],x2:b[0]+c,y2:b[1]},style:{stroke:'%s'}}]};}" % (cap, color, color, color))
        return self._custom(name, [[x, lo, hi] for x, lo, hi in zip(xs, lows, highs)], js)

    def add_errorbar_series_symmetric(self, name, xs, ys, yerr, color="#333", cap=4):
        return self.add_errorbar_series(name, xs, [y - e for y, e in zip(ys, yerr)], [y + e for y, e in zip(ys, yerr)],
                                        color, cap)

    def add_eventplot_series_horizontal(self, name, events, color="#1f77b4", line_len=18):
        data = [[t, r] for r, row in enumerate(events) for t in row]
        return self._add("scatter", name, data, symbol="rect", symbolSize=[2, line_len], itemStyle={"color": color})

    def add_hexbin_series_from_bins(self, name, centers, values, size=20):
        return self._add("scatter", name, [[c[0], c[1], v] for c, v in zip(centers, values)], symbolSize=size,
                         symbol="path://M0,-1L0.866,-0.5L0.866,0.5L0,1L-0.866,0.5L-0.866,-0.5Z")

    def add_quiver_series(self, name, xs, ys, u, v, scale=1.0, color="#1f77b4"):
        js = ("function(p,api){var a=api.coord([api.value(0),api.value(1)]),b=api.coord([api.value(2),api.value(3)]);"
              "var t=Math.atan2(b[1]-a[1],b[0]-a[0]),h=6;return {type:'group',children:["
              "{type:'line',shape:{x1:a[0],y1:a[1],x2:b[0],y2:b[1]},style:{stroke:'%s'}},"
              "{type:'polygon',shape:{points:[[b[0],b[1]],[b[0]-h*Math.cos(t-0.4),b[1]-h*Math.sin(t-0.4)],"
              "[b[0]-h*Math.cos(t+0.4),b[1]-h*Math.sin(t+0.4)]]},style:{fill:'%s'}}]};}" % (color, color))
        return self._custom(name, [[x, y, x + a * scale, y + b * scale] for x, y, a, b in zip(xs, ys, u, v)], js)

    def add_sankey_series(self, name, nodes, links, orient="horizontal"):
        s = {"type": "sankey", "name": name, "orient": orient, "data": [{"name": n} for n in nodes],
             "links": [{"source": a, "target": b, "value": v} for a, b, v in links]}
        self.series.append(s); return self

    # ---- polar ----
    def set_polar(self, center=("50%", "55%"), radius="70%"):
        self.o["polar"] = {"center": list(center), "radius": radius}; return self

    def set_angle_axis_value(self, minv=0, maxv=360, start_angle=90, clockwise=True):
        self.o["angleAxis"] = {"type": "value", "min": minv, "max": maxv, "startAngle": start_angle,
                               "clockwise": bool(clockwise)}
        return self

    def set_radius_axis_value(self, minv=None, maxv=None, name=""):
        a = {"type": "value", "name": name}
        if minv is not None:
            a["min"] = minv
        if maxv is not None:
            a["max"] = maxv
        self.o["radiusAxis"] = a; return self

    set_radius_axis_value_json = set_radius_axis_value

    def set_angle_axis_category(self, categories, start_angle=90):
        self.o["angleAxis"] = {"type": "category", "data": list(categories), "startAngle": start_angle}; return self

    set_angle_axis_category_json = set_angle_axis_category

    def set_polar_axes_value(self, rmin=None, rmax=None):
        self.set_polar()
        self.set_angle_axis_value()
        return self.set_radius_axis_value(rmin, rmax)

    def _polar(self, kind, name, theta, r, **kw):
        return self._add(kind, name, [[rr, t] for t, rr in zip(theta, r)], coordinateSystem="polar", **kw)

    def add_polar_scatter_series(self, name, theta, r, color=None, symbol_size=8):
        return self._polar("scatter", name, theta, r, symbolSize=symbol_size, itemStyle={"color": color} if color else None)

    def add_polar_line_series(self, name, theta, r, color=None, smooth=False):
        return self._polar("line", name, theta, r, smooth=bool(smooth), showSymbol=False,
                           itemStyle={"color": color} if color else None)

    def add_polar_bar_series(self, name, values, color=None, stack=None):
        return self._add("bar", name, list(values), coordinateSystem="polar", stack=stack,
                         itemStyle={"color": color} if color else None)

    # ---- 3-D ----
    def _axis3d(self, key, name, name_gap, axis_color):
        self.o[key] = {"type": "value", "name": name, "nameGap": name_gap, "axisLine": {"lineStyle": {"color": axis_color}}}
        return self

    def set_xaxis3d_value(self, name, name_gap=20, axis_color="#999"): return self._axis3d("xAxis3D", name, name_gap, axis_color)
    def set_yaxis3d_value(self, name, name_gap=20, axis_color="#999"): return self._axis3d("yAxis3D", name, name_gap, axis_color)
    def set_zaxis3d_value(self, name, name_gap=20, axis_color="#999"): return self._axis3d("zAxis3D", name, name_gap, axis_color)

    def set_grid3d_default(self, box_width=100, box_depth=100, box_height=60, auto_rotate=False):
        self.o["grid3D"] = {"boxWidth": box_width, "boxDepth": box_depth, "boxHeight": box_height,
                            "viewControl": {"autoRotate": bool(auto_rotate)}}
        return self

    def add_surface3d_series(self, name, rows, cols, zvals, wireframe=True):
        z = list(zvals)
        data = [[c, r, z[r * cols + c]] for r in range(rows) for c in range(cols) if r * cols + c < len(z)]
        return self._add("surface", name, data, dataShape=[rows, cols], wireframe={"show": bool(wireframe)})

    # ---- calendar / single axis ----
    def set_calendar_json(self, calendar_json):
        self.o["calendar"] = _frag(calendar_json); return self

    def set_calendar_simple(self, range_str, top=120, left=40, right=40, cell_size=("auto", 18)):
        self.o["calendar"] = {"range": range_str, "top": top, "left": left, "right": right, "cellSize": list(cell_size)}
        return self

    def add_calendar_heatmap_series(self, name, items):
        return self._add("heatmap", name, [[d, v] for d, v in items], coordinateSystem="calendar")

    def set_single_axis_time(self, top=60, bottom=60, name=""):
        self.o["singleAxis"] = {"type": "time", "top": top, "bottom": bottom, "name": name}; return self

    def add_theme_river_series(self, name, rows):
        return self._add("themeRiver", name, [list(r) for r in rows])

    # ---- part-of-whole / hierarchical ----
    def add_funnel_series(self, name, labels, values, sort="descending", gap=2, left="10%", width="80%"):
        return self._add("funnel", name, [{"name": n, "value": v} for n, v in zip(labels, values)], sort=sort, gap=gap,
                         left=left, width=width)

    def add_gauge_series(self, name, value, minv=0, maxv=100, unit="%", title=""):
        return self._add("gauge", name, [{"value": value, "name": title or name}], min=minv, max=maxv,
                         detail={"formatter": "{value}" + unit})

    def add_map_choropleth(self, name, pairs, map_name="world", roam=True):
        return self._add("map", name, [{"name": n, "value": v} for n, v in pairs], map=map_name, roam=bool(roam))

    def set_parallel_layout(self, left="5%", right="13%", bottom="10%", top="20%"):
        self.o["parallel"] = {"left": left, "right": right, "bottom": bottom, "top": top}; return self

    def add_parallel_axis(self, dim, name, axis_type="value", categories=None):
        a = {"dim": dim, "name": name, "type": axis_type}
        if categories:
            a["data"] = list(categories)
        self.parallel_axes.append(a); return self

    def add_parallel_series_int(self, name, rows, color=None, width=1):
        return self._add("parallel", name, [list(r) for r in rows],
                         lineStyle={"width": width, **({"color": color} if color else {})})

    add_parallel_series = add_parallel_series_int

    def set_radar_from_names_maxes(self, names, maxes, shape="polygon"):
        self.o["radar"] = {"shape": shape, "indicator": [{"name": n, "max": m} for n, m in zip(names, maxes)]}
        return self

    def add_radar_series(self, name, rows, row_names=None, area=False):
        row_names = row_names or [f"{name} {i + 1}" for i in range(len(rows))]
        return self._add("radar", name, [{"name": n, "value": list(r)} for n, r in zip(row_names, rows)],
                         areaStyle={} if area else None)

    def sb_node(self, name, value=0, children=None) -> str:
        n = {"name": name}
        if value:
            n["value"] = value
        if children:
            n["children"] = [_frag(c) for c in children]
        return dumps(n)

    build_tree_node = sb_node

    def add_sunburst_series(self, name, nodes, radius=(0, "90%")):
        return self._add("sunburst", name, [_frag(n) for n in nodes], radius=list(radius))

    def build_treemap_flat(self, labels, values) -> str:
        return dumps([{"name": n, "value": v} for n, v in zip(labels, values)])

    def add_treemap_series(self, name, data, leaf_depth=None):
        return self._add("treemap", name, _frag(data), leafDepth=leaf_depth)

    def add_tree_series(self, name, root, orient="LR", symbol_size=8):
        return self._add("tree", name, [_frag(root)], orient=orient, symbolSize=symbol_size,
                         label={"position": "left", "verticalAlign": "middle", "align": "right"})

    def add_wordcloud_series(self, name, words, sizes=(12, 60), shape="circle"):
        return self._add("wordCloud", name, [{"name": w, "value": v} for w, v in words], shape=shape,
                         sizeRange=list(sizes))

    # ---- output ----
    def to_dict(self) -> dict:
        out = dict(self.o)
        if self.titles:
            out["title"] = self.titles if len(self.titles) > 1 else self.titles[0]
        if self.datazoom:
            out["dataZoom"] = list(self.datazoom)
        if self.parallel_axes:
            out["parallelAxis"] = list(self.parallel_axes)
        out["series"] = list(self.series)
        return out

    def to_json(self) -> str:
        s = dumps(self.to_dict())
        # custom-series render functions travel as marked strings and are unquoted here
        while '"@@' in s:
            a = s.index('"@@')
            b = s.index('@@"', a)
            s = s[:a] + loads('"' + s[a + 3:b] + '"') + s[b + 3:]
        if self.extra:
            s = s[:-1] + ("," if len(s) > 2 else "") + ",".join(self.extra) + "}"
        return s
