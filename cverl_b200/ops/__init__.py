"""Hot ops: hand-written sm_100a kernels behind autograd functions, each with a PyTorch oracle."""
from .gemm import gemm_nn, gemm_nt, gemm_tn_acc, linear, launch_counter  # noqa: F401
from .norm import add_rmsnorm, gated_rmsnorm, headnorm_rope, rmsnorm, rope_tables  # noqa: F401
from .activation import conv1d_silu, conv1d_silu_split, embedding, siggate, swiglu  # noqa: F401
from .lmhead import lmhead_logprob  # noqa: F401
from . import rl, optim  # noqa: F401
