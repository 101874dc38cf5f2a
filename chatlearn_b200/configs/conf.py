"""A small YAML → dataclass configuration resolver.

The reference composes its config with Hydra + OmegaConf
(chatlearn/entrypoint.py:87-103): structured dataclass schema, an external
YAML file merged on top, ``key.sub=value`` dot-list overrides, ``${a.b}``
interpolation and ``MISSING`` sentinels.  Neither library is a dependency
here; this module implements exactly that subset:

* ``load_yaml`` / ``merge`` / ``apply_dotlist`` on plain nested dicts,
* ``resolve`` for ``${path.to.key}``, ``${oc.env:NAME,default}`` and the legacy
  ``${NAME:default}`` environment form (chatlearn/utils/arguments.py:46-98),
* ``to_dataclass`` which instantiates a (possibly nested) dataclass schema from
  the resolved dict with type coercion and reports unknown / missing keys.
"""
import dataclasses
import os
import re
import typing
from typing import Any, Dict, List, Optional, Union

import yaml


class _Missing:
    _inst = None

    def __new__(cls):
        if cls._inst is None:
            cls._inst = super().__new__(cls)
        return cls._inst

    def __repr__(self):
        return "???"

    def __bool__(self):
        return False


MISSING = _Missing()


class ConfigError(ValueError):
    pass


_yaml_loader = yaml.SafeLoader
# YAML 1.1 does not read "2e-6" as float; accept it like OmegaConf does.
_yaml_loader.add_implicit_resolver(
    "tag:yaml.org,2002:float",
    re.compile(r"""^[-+]?(?:[0-9][0-9_]*\.[0-9_]*(?:[eE][-+]?[0-9]+)?
                    |[0-9][0-9_]*[eE][-+]?[0-9]+
                    |\.[0-9_]+(?:[eE][-+]?[0-9]+)?
                    |\.(?:inf|Inf|INF)|\.(?:nan|NaN|NAN))$""", re.X),
    list("-+0123456789."))


def load_yaml(path_or_text: str, is_text=False) -> Dict[str, Any]:
    if is_text:
        data = yaml.load(path_or_text, Loader=_yaml_loader)
        return data or {}
    with open(path_or_text, "r", encoding="utf-8") as f:
        data = yaml.load(f, Loader=_yaml_loader) or {}
    base = os.path.dirname(os.path.abspath(path_or_text))
    # legacy ``includes: [a.yaml, b.yaml]`` merging (arguments.py:350-539)
    inc = data.pop("includes", None)
    if inc:
        merged = {}
        for p in inc:
            merged = merge(merged, load_yaml(p if os.path.isabs(p) else os.path.join(base, p)))
        data = merge(merged, data)
    return data


def merge(base: Dict, over: Dict) -> Dict:
    """Recursive dict merge; values in ``over`` win."""
    out = dict(base)
    for k, v in over.items():
        if k in out and isinstance(out[k], dict) and isinstance(v, dict):
            out[k] = merge(out[k], v)
        else:
            out[k] = v
    return out


def _parse_scalar(text: str):
    try:
        return yaml.load(text, Loader=_yaml_loader)
    except yaml.YAMLError:
        return text


def apply_dotlist(cfg: Dict, dotlist: List[str]) -> Dict:
    """``["a.b=1", "+x.y=[1,2]"]`` → nested assignment (``+`` prefix tolerated)."""
    out = merge({}, cfg)
    for item in dotlist or []:
        if "=" not in item:
            raise ConfigError(f"override '{item}' is not key=value")
        key, val = item.split("=", 1)
        key = key.lstrip("+")
        node = out
        parts = key.split(".")
        for p in parts[:-1]:
            if p not in node or not isinstance(node[p], dict):
                node[p] = {}
            node = node[p]
        node[parts[-1]] = _parse_scalar(val)
    return out


_INTERP = re.compile(r"\$\{([^${}]+)\}")


def _lookup(root: Dict, path: str):
    node = root
    for p in path.split("."):
        if isinstance(node, dict) and p in node:
            node = node[p]
        elif isinstance(node, list) and p.isdigit() and int(p) < len(node):
            node = node[int(p)]
        else:
            raise KeyError(path)
    return node


def _resolve_expr(root, expr: str, stack):
    expr = expr.strip()
    if expr.startswith("oc.env:"):
        body = expr[len("oc.env:"):]
        name, _, default = body.partition(",")
        val = os.environ.get(name.strip())
        if val is None:
            if not _:
                raise ConfigError(f"environment variable {name} is not set")
            return _parse_scalar(default.strip())
        return _parse_scalar(val)
    if ":" in expr and "." not in expr.split(":", 1)[0]:
        # legacy ${ENV_NAME:default}
        name, default = expr.split(":", 1)
        val = os.environ.get(name.strip())
        return _parse_scalar(val if val is not None else default.strip())
    if expr in stack:
        raise ConfigError(f"interpolation cycle at ${{{expr}}}")
    try:
        val = _lookup(root, expr)
    except KeyError:
        env = os.environ.get(expr)
        if env is not None:
            return _parse_scalar(env)
        raise ConfigError(f"interpolation key '{expr}' not found") from None
    return _resolve_value(root, val, stack + (expr,))


def _resolve_value(root, val, stack=()):
    if isinstance(val, str):
        m = _INTERP.fullmatch(val.strip())
        if m:
            return _resolve_expr(root, m.group(1), stack)
        prev = None
        while prev != val and _INTERP.search(val):
            prev = val
            val = _INTERP.sub(lambda mm: str(_resolve_expr(root, mm.group(1), stack)), val)
        return val
    if isinstance(val, dict):
        return {k: _resolve_value(root, v, stack) for k, v in val.items()}
    if isinstance(val, list):
        return [_resolve_value(root, v, stack) for v in val]
    return val


def resolve(cfg: Dict) -> Dict:
    """Resolve every ``${...}`` in ``cfg`` against ``cfg`` itself."""
    return _resolve_value(cfg, cfg)


# --------------------------------------------------------------------------
# dict -> dataclass
# --------------------------------------------------------------------------

def _coerce(tp, val, path):
    if val is MISSING or val is None:
        return val
    origin = typing.get_origin(tp)
    if tp is Any or tp is None:
        return val
    if origin is Union:
        args = [a for a in typing.get_args(tp) if a is not type(None)]
        last = None
        for a in args:
            try:
                return _coerce(a, val, path)
            except (ConfigError, TypeError, ValueError) as e:  # try next arm
                last = e
        raise ConfigError(f"{path}: cannot coerce {val!r} to {tp}: {last}")
    if origin in (list, List):
        (et,) = typing.get_args(tp) or (Any,)
        if isinstance(val, str):
            val = _parse_scalar(val)
        if not isinstance(val, (list, tuple)):
            raise ConfigError(f"{path}: expected list, got {val!r}")
        return [_coerce(et, v, f"{path}[{i}]") for i, v in enumerate(val)]
    if origin in (dict, Dict):
        if not isinstance(val, dict):
            raise ConfigError(f"{path}: expected dict, got {val!r}")
        return dict(val)
    if dataclasses.is_dataclass(tp):
        if dataclasses.is_dataclass(val):
            return val
        if not isinstance(val, dict):
            raise ConfigError(f"{path}: expected mapping for {tp.__name__}, got {val!r}")
        return to_dataclass(tp, val, path)
    if tp is bool:
        if isinstance(val, bool):
            return val
        if isinstance(val, str) and val.lower() in ("true", "false", "1", "0", "yes", "no"):
            return val.lower() in ("true", "1", "yes")
        if isinstance(val, int):
            return bool(val)
        raise ConfigError(f"{path}: expected bool, got {val!r}")
    if tp is int:
        if isinstance(val, bool):
            return int(val)
        if isinstance(val, int):
            return val
        if isinstance(val, float) and val == int(val):
            return int(val)
        if isinstance(val, str):
            return int(val)
        raise ConfigError(f"{path}: expected int, got {val!r}")
    if tp is float:
        if isinstance(val, (int, float)) and not isinstance(val, bool):
            return float(val)
        if isinstance(val, str):
            return float(val)
        raise ConfigError(f"{path}: expected float, got {val!r}")
    if tp is str:
        return val if isinstance(val, str) else str(val)
    return val


def to_dataclass(cls, data: Optional[Dict], path: str = "", strict: bool = False):
    """Instantiate dataclass ``cls`` from ``data``.

    Unknown keys are kept as plain attributes unless ``strict`` (reference YAMLs
    carry engine-specific extras such as ``vllm_prompt_key``)."""
    data = data or {}
    hints = typing.get_type_hints(cls)
    kwargs, extras = {}, {}
    names = {f.name for f in dataclasses.fields(cls) if f.init}
    for k, v in data.items():
        if k in names:
            kwargs[k] = _coerce(hints.get(k, Any), v, f"{path}.{k}" if path else k)
        elif strict:
            raise ConfigError(f"{path or cls.__name__}: unknown key '{k}'")
        else:
            extras[k] = v
    obj = cls(**kwargs)
    for k, v in extras.items():
        setattr(obj, k, v)
    return obj


def missing_keys(obj, path="") -> List[str]:
    """Dotted paths of fields still equal to ``MISSING``."""
    out = []
    if dataclasses.is_dataclass(obj):
        for f in dataclasses.fields(obj):
            v = getattr(obj, f.name)
            p = f"{path}.{f.name}" if path else f.name
            if v is MISSING:
                out.append(p)
            else:
                out.extend(missing_keys(v, p))
    elif isinstance(obj, dict):
        for k, v in obj.items():
            out.extend(missing_keys(v, f"{path}.{k}" if path else str(k)))
    return out


def to_container(obj):
    """dataclass / nested containers → plain dict (for dumps and checkpoints)."""
    if dataclasses.is_dataclass(obj):
        d = {f.name: to_container(getattr(obj, f.name)) for f in dataclasses.fields(obj)}
        for k, v in vars(obj).items():
            if k not in d and not k.startswith("_"):
                d[k] = to_container(v)
        return d
    if isinstance(obj, dict):
        return {k: to_container(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [to_container(v) for v in obj]
    if obj is MISSING:
        return "???"
    return obj
