"""Chart emitters produce parseable ECharts options / pages; the ``momijo`` name aliases the package."""
import json
import os

import momijo_b200.visual as U


def test_chart_builders_emit_json():
    opts = [U.chart_line("L", [0, 1, 2], [1, 4, 9], area=True), U.chart_bar("B", ["a", "b"], [1, 2], horizontal=True),
            U.chart_pie("P", ["a", "b"], [1, 2], donut=True), U.chart_heatmap("H", 2, 2, [1, 2, 3, 4]),
            U.chart_boxplot("Bx", [[1, 2, 3, 4, 5], [2, 3, 4]]), U.chart_sankey("S", ["a", "b"], [["a", "b", "3"]]),
            U.chart_surface3d("S3", 2, 2, [0, 1, 2, 3]), U.chart_polar_bar("PB", [0, 90], [1, 2]),
            U.chart_violin("V", ["g"], [[0.1, 0.4, 0.1]], [[0, 1, 2]]), U.chart_eventplot("E", 2, [[1, 2], [3]]),
            U.chart_contour_lines("C", [[[0, 0], [1, 1]]]), U.chart_hexbin("Hx", [[0, 0]], 10, [1], 0, 1),
            U.echarts_bar_option(["x", "y"], [[1, 2], [3, 4]], ["s1", "s2"], stacked=True),
            U.echarts_line_option(["x", "y"], [[1, 2]], ["s"], area=True), U.echarts_scatter_option([1], [2]),
            U.echarts_radar_option([("a", 5), ("b", 5)], [[1, 2]], ["r"]), U.echarts_candlestick_option(["d"], [1], [3], [0], [2]),
            U.echarts_gauge_option(42.0), U.echarts_funnel_option(["a"], [1]), U.echarts_treemap_option(["a"], [1]),
            U.echarts_sunburst_option(["a"], [1]), U.echarts_parallel_option(["p", "q"], [[1, 2]]),
            U.echarts_calendar_option("2024", [("2024-01-01", 1.0)]), U.echarts_heatmap_option(["a"], ["b"], [[1.0]]),
            U.echarts_themeriver_option(["2024-01-01"], ["n"], [[1.0]]), U.echarts_map_option([("X", 1.0)]),
            U.echarts_sankey_option(["a", "b"], [("a", "b", 1.0)]), U.echarts_pictorialbar_option(["a"], [1.0]),
            U.echarts_graph_option(["a", "b"], [(0, 1)]), U.echarts_boxplot_option(["g"], [[1, 2, 3]])]
    for o in opts:
        d = json.loads(o)
        assert "series" in d
    box = json.loads(opts[4])["series"][0]["data"][0]
    assert box == [1, 2, 3, 4, 5]
    assert json.loads(opts[12])["series"][0]["stack"] == "total"
    for o in (U.chart_stem("St", [1], [2]), U.chart_errorbar("Er", [1], [2], [0.1]), U.chart_quiver("Q", [0], [0], [1], [1])):
        assert "function(p,api)" in o
    assert json.loads(U.axis_log(2)) == {"type": "log", "logBase": 2}
    assert json.loads(U.parallel_axis(1, "n"))["dim"] == 1
    assert json.loads(U.visualMap_continuous(0, 1))["type"] == "continuous"


def test_option_assemblers_and_html(tmp_path):
    o = U.Option()
    o.set_title('{"text":"hi"}')
    o.set_xaxis_category(["a", "b"])
    o.set_yaxis_value()
    o.add_series_json(U.series_bar("s", [1, 2]))
    o.add_datazoom_json('{"type":"inside"}')
    o.set_colors(["#f00"])
    d = json.loads(o.to_json())
    assert d["series"][0]["type"] == "bar" and d["dataZoom"][0]["type"] == "inside" and d["color"] == ["#f00"]
    e = U.EasyOption()
    e.set_title("T").set_tooltip_axis_shadow().set_legend(["a"]).set_grid(90, "5%", "5%", "8%")
    e.set_xaxis_category_json("x", "middle", 30, ["p", "q"]).set_yaxis_value_json("y", "middle", 40)
    e.add_bar_series("a", [1, 2], "#f00").add_line_series("b", [2, 3]).add_pie_series("p", ["u"], [1])
    e.add_waterfall_series("w", [3, -1]).add_radar_series("r", [[1, 2]])
    d = json.loads(e.to_json())
    assert d["title"]["text"] == "T" and len(d["series"]) == 7
    e.add_errorbar_series_symmetric("err", [0], [1], [0.1])
    assert "function(p,api)" in e.to_json()
    p = str(tmp_path / "a.html")
    assert U.render_echarts(e.to_json(), p, title="<t>")
    page = open(p, encoding="utf-8").read()
    assert "echarts.init" in page and "&lt;t&gt;" in page
    f = U.new_figure(640, 480, "t", "y")
    f._xs, f._ys, f._names = ["a", "b"], [[1, 2]], ["s"]
    assert U.export_figure_html(f, str(tmp_path / "b.html")) and os.path.getsize(tmp_path / "b.html") > 200
    assert U.get_exporter("nope") is None and U.get_exporter("echarts").name() == "echarts"
    assert "c1" in U.echarts_dashboard_html([opts for opts in ("{}", "{}")], ["a", "b"])


def test_numeric_helpers():
    assert U.hist1d([0.1, 0.5, 0.9, 2.0], 2, 0, 1) == [1, 2]
    assert abs(U.kde_1d([0.0], [0.0], 1.0)[0] - 0.3989) < 1e-3
    segs = U.marching_squares([[0, 0, 0], [0, 1, 0], [0, 0, 0]], 0.5)
    assert len(segs) == 4 and all(len(s) == 2 for s in segs)
    assert U.json_string('a"b') == '"a\\"b"' and U.json_number_array([1, 2.5]) == "[1,2.5]"


def test_momijo_alias():
    import momijo
    import momijo.learn.nn as nn_alias
    import momijo.tensor as t_alias
    import momijo_b200.learn.nn as nn_real
    import momijo_b200.tensor as t_real
    from momijo.vision import Image
    from momijo.dataframe import DataFrame
    from momijo.visual import echarts_html
    assert nn_alias is nn_real and t_alias is t_real
    assert momijo.learn is __import__("momijo_b200").learn
    assert Image is __import__("momijo_b200.vision", fromlist=["Image"]).Image
    assert DataFrame is not None and callable(echarts_html)
