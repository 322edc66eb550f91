"""momijo.dataframe: pandas-like frames without pandas (CPU only)."""
from .frame import (  # noqa: F401
    DataFrame, Series, Column, Value, Index, MultiIndex, Bitmap, DType, int32, int64, float32, float64,
    string, NaN, NoneStr, isna, series_from_list, Series_from_strings, series_index,
)
from .frame import bool_ as bool  # noqa: F401
from .ops import *  # noqa: F401,F403
from .ops import range, filter, where, copy, rename  # noqa: F401
from . import window, extras, relational  # noqa: F401,E402
from .window import *  # noqa: F401,F403,E402
from .extras import *  # noqa: F401,F403,E402
from .relational import *  # noqa: F401,F403,E402
from .relational import eval, get  # noqa: F401,E402
from .ops import range, filter, where, copy, rename  # noqa: F401,E402,F811
from .frame import bool_ as bool  # noqa: F401,E402,F811
from . import methods  # noqa: F401,E402  (binds the method spellings onto the classes above)

int32, int64, float32, float64, string = (methods.DTYPE_CONSTRUCTORS[n] for n in ("int32", "int64", "float32", "float64", "string"))
bool_ = methods.DTYPE_CONSTRUCTORS["bool"]

from .. import _layout as _layout  # noqa: E402

_layout.link_siblings("dataframe")   # names the reference keeps in another file of this package still resolve
