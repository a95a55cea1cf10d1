from .types import Err, Ok, Result, flat_map, is_err, is_ok, map_err, map_result, unwrap, unwrap_err, unwrap_or, unwrap_or_else  # noqa: F401
from .errors import *  # noqa: F401,F403
