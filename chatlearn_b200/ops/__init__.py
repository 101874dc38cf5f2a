"""Op facade used by the models, trainers and the rollout engine.

Device decides the implementation: CPU tensors run the PyTorch statements in
``ops.reference`` (plumbing runs and oracles); CUDA tensors run the hand-written
sm_100a kernels from the in-tree extension (``ops.native``).  ``set_mode
("library")`` routes CUDA tensors to the PyTorch/cuBLAS statements instead: that
is the baseline the kernels are measured against, not a fallback — in native
mode a CUDA tensor with no loadable extension raises.
"""
import contextlib
from collections import Counter

import torch

from . import reference as ref

_MODE = "native"
_NATIVE = {}
launch_counts = Counter()      # native kernel launches by op name (bench reports the sum)
library_counts = Counter()     # CUDA calls that ran a library statement in native mode


def set_mode(mode: str):
    global _MODE
    assert mode in ("native", "library")
    _MODE = mode


def get_mode() -> str:
    return _MODE


@contextlib.contextmanager
def mode(m: str):
    prev = _MODE
    set_mode(m)
    try:
        yield
    finally:
        set_mode(prev)


def register_native(name, fn):
    _NATIVE[name] = fn


def native_ops():
    return sorted(_NATIVE)


_native_loaded = None


def _ensure_native():
    global _native_loaded
    if _native_loaded is None:
        from . import native  # noqa: F401  (registers kernels; raises if the .so is missing)
        _native_loaded = True


def _use_native(name, t: torch.Tensor) -> bool:
    if not t.is_cuda or _MODE != "native":
        return False
    _ensure_native()
    if name in _NATIVE:
        return True
    library_counts[name] += 1
    return False


def _dispatch(name):
    r = getattr(ref, name)

    def op(*args, **kwargs):
        t = next(a for a in args if isinstance(a, torch.Tensor))
        if _use_native(name, t):
            return _NATIVE[name](*args, **kwargs)
        return r(*args, **kwargs)
    op.__name__ = name
    op.__doc__ = r.__doc__
    return op


rmsnorm = _dispatch("rmsnorm")
add_rmsnorm_ = _dispatch("add_rmsnorm_")
swiglu = _dispatch("swiglu")
linear = _dispatch("linear")
linear_planes = _dispatch("linear_planes")
rope = _dispatch("rope")
rope_mrope = _dispatch("rope_mrope")
qk_norm_rope = _dispatch("qk_norm_rope")
qkv_rope_append = _dispatch("qkv_rope_append")
attention_varlen = _dispatch("attention_varlen")
attention_segments = _dispatch("attention_segments")
kv_append = _dispatch("kv_append")
paged_attention = _dispatch("paged_attention")
mla_paged_decode = _dispatch("mla_paged_decode")
lmhead_logprob_entropy = _dispatch("lmhead_logprob_entropy")
grpo_loss_fused = _dispatch("grpo_loss_fused")
gspo_loss_fused = _dispatch("gspo_loss_fused")
adamw_step = _dispatch("adamw_step")
sumsq = _dispatch("sumsq")
moe_router = _dispatch("moe_router")
moe_experts = _dispatch("moe_experts")
grouped_mlp = _dispatch("grouped_mlp")
sample = _dispatch("sample")
apply_penalties = _dispatch("apply_penalties")

# pure-PyTorch helpers with no kernel counterpart
grpo_token_loss = ref.grpo_token_loss
gspo_token_loss = ref.gspo_token_loss
kl_k3 = ref.kl_k3
moe_aux_loss = ref.moe_aux_loss
logprobs_from_logits = ref.logprobs_from_logits
entropy_from_logits = ref.entropy_from_logits
rope_cos_sin = ref.rope_cos_sin
