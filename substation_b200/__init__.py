"""substation_b200: the BERT encoder-layer forward+backward of spcl/substation's
``pytorch_module/encoder.py``, rebuilt for B200 (sm_100a).

``Encoder`` is the drop-in module; ``ops`` exposes each fused kernel and the
contraction kernel on their own; ``layouts`` holds the layout-configuration
contract.  The CUDA library is loaded on first use and there is no fallback
when it is missing.
"""

from . import layouts  # noqa: F401
from .encoder import Encoder  # noqa: F401

__all__ = ['Encoder', 'layouts', 'ops']


def __getattr__(name):
    if name == 'ops':
        import importlib
        return importlib.import_module('.ops', __name__)
    raise AttributeError(name)
