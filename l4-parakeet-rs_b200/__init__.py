"""B200 (sm_100a) kernels for the FastConformer / TDT hot path of l4-parakeet-rs.

`lib` is the ctypes view of the C ABI (include/pk100.h); `ops` wraps it for
torch CUDA tensors (device memory and streams only -- no torch arithmetic).
"""
from . import lib  # noqa: F401  (raises if libpk100.so is not built)
from . import ops  # noqa: F401
from . import encoder  # noqa: F401
from . import synth  # noqa: F401
from . import decoder  # noqa: F401
from . import subsampling  # noqa: F401
from . import pipeline  # noqa: F401
from . import parallel  # noqa: F401
from . import artifact  # noqa: F401
from . import frontend  # noqa: F401
