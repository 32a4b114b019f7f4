"""B200-native ops for the attention code Mercury's CommIR PyTorch backend emits."""
from . import _lib  # noqa: F401  (fails loudly when libmercury_b200.so is missing)
from .attention import (attn_bwd_dkv, attn_bwd_dq, attn_bwd_fused, attn_fwd_multi, attn_fwd_segments,  # noqa: F401
                        bwd_preprocess)
from .integration import (install_backend, install_search_hooks, load_generated, namespace,  # noqa: F401
                          remove_search_hooks)
from .ops import (_flash_attn_backward, _flash_attn_forward, flash_reduce, get_default_args,  # noqa: F401
                  update_out_and_lse)
