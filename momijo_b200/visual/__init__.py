"""Chart package: ECharts option JSON and standalone HTML pages as text. Public names follow the
reference's aggregate import list (legacy/src/momijo/visual/__init__.mojo:6-140). Rendering to pixels
needs a browser, which is outside this package (and absent on GPU servers): files are written, not shown."""
from .core import (dumps, echarts_html, escape_html, json_array_f64, json_array_str, json_number_array,  # noqa: F401
                   json_string, json_string_array, loads, write_text)
from .html import open_in_browser, preview, render_echarts, render_html, write_preview_html  # noqa: F401
from .misc import *  # noqa: F401,F403
from .misc import (ChartExporter, EChartsConfig, EChartsExporter, Figure, export_figure_html, export_html,  # noqa: F401
                   get_exporter, make_echarts_exporter, name, new_figure)
from .option import EasyOption, Option, series_bar, series_line  # noqa: F401
from .plotting import *  # noqa: F401,F403
from .plotting import _compute_violin_curve_json, _ints  # noqa: F401

from .. import _layout as _layout  # noqa: E402

_layout.open_submodules()   # ``visual.core.core``, ``visual.misc.bar`` ... resolve as facades of these modules

_layout.link_siblings("visual")   # names the reference keeps in another file of this package still resolve
