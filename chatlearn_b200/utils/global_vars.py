"""Process-global state: parsed args, decorated-function registry, control deps.

Parity: chatlearn/utils/global_vars.py:30-41 (``get_args``/``set_global_variables``).
"""
_ARGS = None
_EXIT_FLAG = False
_DECORATED = {}
_DEPENDENCIES = None


def set_global_variables(args):
    global _ARGS
    _ARGS = args


def get_args():
    assert _ARGS is not None, "call chatlearn_b200.init(cfg) first"
    return _ARGS


def is_initialized():
    return _ARGS is not None


def reset():
    global _ARGS, _DEPENDENCIES
    _ARGS = None
    _DEPENDENCIES = None
    _DECORATED.clear()


def set_decorated(model_name):
    _DECORATED[model_name] = True


def is_decorated(model_name):
    return _DECORATED.get(model_name, False)


def set_dependencies(deps):
    global _DEPENDENCIES
    _DEPENDENCIES = deps


def get_dependencies():
    return _DEPENDENCIES


def reset_dependencies():
    global _DEPENDENCIES
    _DEPENDENCIES = None
