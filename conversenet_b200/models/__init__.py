"""Network definitions with the reference's class names, constructor signatures and
state-dict keys (`models/converse_dncnn.py`, `models/converse_srresnet.py`,
`models/converse_usrnet.py`), built on the native Converse2D / ConverseBlock."""
from .converse_dncnn import ConverseDnCNN  # noqa: F401
from .converse_srresnet import ConverseMSRResNet  # noqa: F401
from .converse_usrnet import (ConverseUSRNet, ConverseNet, ConvReverseDataNet, KernelNet,  # noqa: F401
                              MultiConverseBlock, MultiConverseBlockAlphaVariant)
