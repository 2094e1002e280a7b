"""`spattn`: the reference's Python operator interface on top of the B200 library.

Importing this package loads the compiled operator module `cuda_attn` (built in-tree from
csrc/extension.cpp), which registers `torch.ops.cuda_attn.*`; there is no fallback if it is absent.
Module and function names follow python/spattn/ of sankeerth95/fgattn_tk_cuda.
"""
import torch  # noqa: F401  (libtorch must be loaded before the extension)

try:
    from . import cuda_attn  # noqa: F401
except ImportError as exc:  # pragma: no cover - build problem, never a silent fallback
    raise ImportError(
        "fgattn_tk_cuda_b200.spattn.cuda_attn is not built; run `python -c \"import __graft_entry__ as g; g.build()\"` "
        "or `python -m fgattn_tk_cuda_b200._build --ext` (no CPU / eager fallback exists)") from exc

from . import mask_utils, sparseattn_functionals  # noqa: E402,F401
