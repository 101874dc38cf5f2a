"""Result resolution helpers.

Parity: chatlearn/utils/future.py:50-91 (``wait`` with a progress bar over Ray
object refs, recursive ``get``).  Calls are local and synchronous here, so a
"future" is either a plain value or a ``concurrent.futures.Future`` (the rollout
manager's asynchronous requests); ``get`` resolves both, recursively."""
from concurrent.futures import Future
from typing import Any


def get(data: Any):
    if isinstance(data, Future):
        return get(data.result())
    if isinstance(data, (list, tuple)):
        return type(data)(get(d) for d in data)
    if isinstance(data, dict):
        return {k: get(v) for k, v in data.items()}
    return data


def wait(refs, desc: str = None, return_output: bool = False):
    if not isinstance(refs, (list, tuple)):
        refs = [refs]
    out = [get(r) for r in refs]
    return out if return_output else None
