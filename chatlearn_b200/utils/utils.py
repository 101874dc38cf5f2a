"""Small shared helpers.

Parity: chatlearn/utils/utils.py:42-445 (``even_slice``, ``split_index``,
``slice_data_list_by_index``, ``to_device``, ``map_reduce_metrics``,
``parse_function_return_num``, memory reports).
"""
import ast
import inspect
import socket
import textwrap
from typing import Any, Dict, List, Sequence

import torch


def even_slice(total_sample: int, total_slice: int) -> List[int]:
    """Boundaries that split ``total_sample`` items into ``total_slice`` nearly
    equal contiguous chunks; the first ``total_sample % total_slice`` chunks get
    one extra item.  Returns ``total_slice + 1`` offsets."""
    assert total_slice > 0
    base, extra = divmod(total_sample, total_slice)
    out = [0]
    for i in range(total_slice):
        out.append(out[-1] + base + (1 if i < extra else 0))
    return out


def split_index(length: int, num_splits: int):
    """(start, end) index pairs of an even split."""
    b = even_slice(length, num_splits)
    return [(b[i], b[i + 1]) for i in range(num_splits)]


def slice_by_index(data, start, end):
    if isinstance(data, torch.Tensor):
        return data[start:end]
    if isinstance(data, (list, tuple)):
        return data[start:end]
    if isinstance(data, dict):
        return {k: slice_by_index(v, start, end) for k, v in data.items()}
    raise TypeError(type(data))


def slice_data_list_by_index(batched_input: Sequence, index):
    """``index = (i, n)``: return the i-th of n even chunks of ``batched_input``."""
    i, n = index
    b = even_slice(len(batched_input), n)
    return batched_input[b[i]:b[i + 1]]


def to_device(device, obj):
    """Recursively move tensors in nested containers to ``device``."""
    if isinstance(obj, torch.Tensor):
        return obj.to(device, non_blocking=True) if obj.device != torch.device(device) else obj
    if isinstance(obj, dict):
        return {k: to_device(device, v) for k, v in obj.items()}
    if isinstance(obj, list):
        return [to_device(device, v) for v in obj]
    if isinstance(obj, tuple):
        return tuple(to_device(device, v) for v in obj)
    return obj


def map_reduce_metrics(metric_list: List[Dict[str, Any]]) -> Dict[str, float]:
    """Mean of every scalar key over a list of metric dicts."""
    acc, cnt = {}, {}
    for m in metric_list:
        for k, v in m.items():
            if isinstance(v, torch.Tensor):
                v = v.float().mean().item()
            if isinstance(v, (list, tuple)):
                if not v:
                    continue
                v = float(sum(v)) / len(v)
            acc[k] = acc.get(k, 0.0) + float(v)
            cnt[k] = cnt.get(k, 0) + 1
    return {k: acc[k] / cnt[k] for k in acc}


def parse_function_return_num(func) -> int:
    """Number of values a flow function returns (0 if it has no ``return``)."""
    src = textwrap.dedent(inspect.getsource(func))
    tree = ast.parse(src)
    fn = tree.body[0]
    nums = []

    class V(ast.NodeVisitor):
        def __init__(self):
            self.depth = 0

        def visit_FunctionDef(self, node):
            self.depth += 1
            if self.depth == 1:
                self.generic_visit(node)
            self.depth -= 1

        visit_AsyncFunctionDef = visit_FunctionDef
        visit_Lambda = lambda self, node: None  # noqa: E731

        def visit_Return(self, node):
            if node.value is None:
                nums.append(0)
            elif isinstance(node.value, ast.Tuple):
                nums.append(len(node.value.elts))
            else:
                nums.append(1)

    V().visit(fn)
    return max(nums) if nums else 0


def get_free_port(addr="127.0.0.1") -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind((addr, 0))
        return s.getsockname()[1]


def device_memory_report(device=None) -> Dict[str, float]:
    """Allocated / reserved / free / total GiB of the current CUDA device."""
    if not torch.cuda.is_available():
        return {}
    free, total = torch.cuda.mem_get_info(device)
    gib = float(1 << 30)
    return {
        "allocated_gib": torch.cuda.memory_allocated(device) / gib,
        "reserved_gib": torch.cuda.memory_reserved(device) / gib,
        "peak_allocated_gib": torch.cuda.max_memory_allocated(device) / gib,
        "free_gib": free / gib,
        "total_gib": total / gib,
    }


def flatten(xs):
    out = []
    for x in xs:
        if isinstance(x, (list, tuple)):
            out.extend(flatten(x))
        else:
            out.append(x)
    return out


def dict_to_simplenamespace(d):
    from types import SimpleNamespace
    if isinstance(d, dict):
        return SimpleNamespace(**{k: dict_to_simplenamespace(v) for k, v in d.items()})
    return d
