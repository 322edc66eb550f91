"""Two charts and a dashboard page written as standalone HTML (the reference's visual demos emit the same
kind of files; opening them needs a browser)."""
import os
import tempfile

import momijo.visual as U


def main(out_dir: str = None):
    out_dir = out_dir or tempfile.mkdtemp()
    line = U.chart_line("squares", [0, 1, 2, 3], [0, 1, 4, 9], area=True)
    bars = U.echarts_bar_option(["q1", "q2"], [[3, 5], [4, 2]], ["north", "south"], stacked=True, title="sales")
    assert U.render_echarts(line, os.path.join(out_dir, "line.html"), title="line")
    page = U.echarts_dashboard_html([line, bars], ["line", "bars"])
    assert U.write_text(os.path.join(out_dir, "dashboard.html"), page)
    print("wrote", sorted(os.listdir(out_dir)))
    return out_dir


if __name__ == "__main__":
    main()
