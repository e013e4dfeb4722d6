"""
RF: the model-definition API. ``import returnn_b200.frontend as rf``.

Modules (:class:`Module`, :class:`Parameter`, layers, encoder/decoder zoo) and functional ops on named-dimension
:class:`Tensor` objects. Execution is eager torch; hot ops dispatch to the sm_100a kernels in
:mod:`returnn_b200.ops` when the tensors live on a B200.

Parity: returnn/frontend/__init__.py (same public names).
"""

from ..tensor import Tensor, Dim, batch_dim, single_step_dim, TensorDict
from ..utils.basic import NotSpecified

from ._utils import RawTensorTypes
from .dtype import *
from .device import *
from .module import *
from .parameter import *
from .container import *
from .state import *
from .run_ctx import *
from .math_ import *
from .array_ import *
from .reduce import *
from .matmul import *
from .dims import *
from .const import *
from .rand import *
from .dropout import *
from .gradient import *
from .cond import *
from .loop import *
from .tensor_array import *
from .label_smoothing import *
from .loss import *
from .signal import *
from .linear import *
from .conv import *
from .normalization import *
from .rec import *
from .attention import *
from .hooks import *
from .parametrize import *
from .build_from_dict import *
from .piecewise_linear import *
from .amp import *
from .static_traceable import *
from .graph import *
from .assert_ import *
from .types import GetModelFunc, StepFunc, ItemKeyType, get_raw_tensor_type
from .backend import select_backend, get_selected_backend, select_backend_numpy, select_backend_tf, is_backend_raw_tensor_dim_tag_independent
from .packed import pack, unpack, pack_import, is_packed, PackedTensor, packed_regap, packed_flat_content

from . import init
from . import nested
from . import audio
from . import encoder
from . import decoder
from . import conversions
from . import hooks
from . import packed
from . import amp
from . import static_traceable
from . import graph
from . import types
from . import backend
from . import stepwise_scheduler
from . import parametrize as parametrizations  # weight dropout / noise live in the parametrize module here
from . import control_flow as _control_flow
from .control_flow import control_flow_ctx, get_current_control_flow_ctx
from .backend_select import select_backend_torch, select_backend_returnn_layers_tf, is_executing_eagerly, get_backend_name

from . import checkpoint  # noqa: E402,F401
from ._random_journal import RandomJournal  # noqa: E402,F401

set_random_seed(42)

# native dimension bookkeeping when the extension is built (RETURNN_B200_RF_NATIVE=0 keeps the Python versions)
from . import _native as _native_opt  # noqa: E402

_native_opt.setup()
