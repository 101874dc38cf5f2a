from .arch import PRESETS, ModelArch, resolve_arch
from .layout import Leaf, Segment, hf_tensor_shapes, model_blocks
from .model import CausalLM, FwdCtx, KVCtx, ParamBlock, decoder_layer, packed_ctx
