"""B200-native execution backend for the Accelerate array language (hot path only).

``accelerate_b200.language`` mirrors the reference's operator interface and
produces the post-fusion program text; ``accelerate_b200.backend`` runs it on
the GPU through the C-ABI library.  Names that collide with Python builtins
carry a trailing underscore inside ``language`` and are re-exported here under
the reference's own names.
"""
from . import language
from .language import *  # noqa: F401,F403
from .language import map_ as map, zip_ as zip, sum_ as sum  # noqa: A001,F401
