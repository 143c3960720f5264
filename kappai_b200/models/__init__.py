"""Built-in architectures.  Importing this package registers them."""
from . import lfm2  # noqa: F401
from . import tizusun  # noqa: F401
from . import vekuzen  # noqa: F401
from . import tupalorn  # noqa: F401
from . import vumotar  # noqa: F401
