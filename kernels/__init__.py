"""Import alias so code written against the reference's layout (`from kernels import kvskip`)
resolves to the sm_100a implementation: `kernels.kvskip` IS the module `kvskip_b200.kvskip` (one
module object under two names, so there is one loaded extension and one set of module globals)."""
import sys

from kvskip_b200 import kvskip

sys.modules[__name__ + ".kvskip"] = kvskip
