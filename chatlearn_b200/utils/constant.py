"""Shared constants.

Parity: chatlearn/utils/constant.py (REF_LIST, INDEX_TAG, LOG_START) and the
string enums scattered across chatlearn/utils/constant.py.
"""

LOG_START = ">>>>>>>>>>>"
REF_LIST = "__ref_list__"
INDEX_TAG = "__index_tag__"

# backends
TRAIN_BACKENDS = ("fsdp", "megatron")
# "native" is this framework's own rollout engine; the historical names are
# accepted as aliases so reference YAML files load unchanged.
ROLLOUT_BACKENDS = ("native", "vllm", "sglang")

# memory tags of the rollout engine (sleep / wake-up granularity)
TAG_WEIGHTS = "weights"
TAG_KV_CACHE = "kv_cache"

# bytes
KiB = 1 << 10
MiB = 1 << 20
GiB = 1 << 30
