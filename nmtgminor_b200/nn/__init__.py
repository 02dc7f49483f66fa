from .blocks import *  # noqa: F401,F403
from .builders import *  # noqa: F401,F403
from .unity import *  # noqa: F401,F403
