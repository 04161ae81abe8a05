"""Built-in architectures.  Importing this package registers them."""

from . import qwen3  # noqa: F401  (first: the default architecture of a model-less run)
from . import logesun  # noqa: F401
from . import puladra  # noqa: F401
from . import medilix  # noqa: F401
from . import tabisun  # noqa: F401
