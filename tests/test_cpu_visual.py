

def test_reference_fragment_spelling_and_field_series():
    """Single-quoted fragments parse; grid heatmap, marching-squares contours, ECDF / survival steps and
    streamlines come out as the series the reference builds."""
    from momijo_b200.visual.core import loads
    from momijo_b200.visual.option import EasyOption, Option
    assert loads("{ 'text':'it\\'s \"a\"', 'n': [1, true, null], \"k\": 'v' }") == {"text": "it's \"a\"", "n": [1, True, None], "k": "v"}
    assert '"title":{"text":"a"}' in Option().set_title("{ 'text':'a' }").set_grid3d_json("{}").to_json()
    e = EasyOption()
    e.set_xaxis_value_json("x", "middle", 20, "#333", "0", "'dataMax'").set_yaxis_category_labels(["a", "b"], "Y")
    e.add_heatmap_series("h", [0, 1], [0, 1], [[1, 2], [3, 4]], 2)
    e.add_contour_lines("c", [0, 1], [0, 1], [[0, 0], [1, 1]], [0.5])
    e.add_ecdf_series("e", [3, 1, 3, 2], "#f00").add_survival_series("s", [3, 1, 3, 2], "#0f0", normalized=False)
    e.add_streamlines_series("st", [[0, 1, 2], [0]], [[0, 1, 0], [1]])
    d = e.to_dict()
    assert d["xAxis"]["max"] == "dataMax" and d["xAxis"]["min"] == 0 and d["yAxis"]["data"] == ["a", "b"]
    by = {s["name"]: s for s in d["series"]}
    assert by["h"]["data"] == [[0, 0, 1], [1, 0, 2], [0, 1, 3], [1, 1, 4]] and by["h"]["blurSize"] == 2
    assert by["c 0.5"]["data"] == [[0, 0.5], [1, 0.5], None]
    assert by["e"]["data"] == [[1, 0.25], [2, 0.5], [3, 1.0]] and by["s"]["data"] == [[1, 3], [2, 2], [3, 0]]
    assert by["st"]["data"] == [{"coords": [[0, 0], [1, 1], [2, 0]]}] and by["st"]["effect"]["trailLength"] == 0.3
