"""
Stand-in for `dataclass_extensions`: a name registry for dataclass hierarchies plus `encode` / `decode` between
dataclasses and plain dicts, sufficient for configs that the benchmark builds in Python.
"""

import dataclasses
import enum
import typing


class Registrable:
    _registry = None
    _default_name = None

    @classmethod
    def _root(cls):
        for base in cls.__mro__:
            if Registrable in base.__bases__:
                return base
        return cls

    @classmethod
    def register(cls, name: str, default: bool = False, exist_ok: bool = True):
        root = cls._root()
        if root.__dict__.get("_registry") is None:
            root._registry = {}

        def deco(sub):
            root._registry[name] = sub
            sub.registered_name = name
            if default:
                root._default_name = name
            return sub

        return deco

    @classmethod
    def get_registered_class(cls, name=None):
        root = cls._root()
        reg = root.__dict__.get("_registry") or {}
        return reg[name if name is not None else root._default_name]

    @classmethod
    def get_registered_name(cls, sub=None):
        return getattr(sub or cls, "registered_name", None)

    @classmethod
    def get_registered_names(cls):
        return list((cls._root().__dict__.get("_registry") or {}).keys())


def encode(obj):
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        return {f.name: encode(getattr(obj, f.name)) for f in dataclasses.fields(obj)}
    if isinstance(obj, enum.Enum):
        return obj.value
    if isinstance(obj, dict):
        return {str(k): encode(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple, set)):
        return [encode(v) for v in obj]
    if isinstance(obj, (str, int, float, bool)) or obj is None:
        return obj
    return str(obj)


def _decode_value(tp, value):
    origin = typing.get_origin(tp)
    if value is None:
        return None
    if origin is typing.Union:
        for arg in typing.get_args(tp):
            if arg is type(None):
                continue
            try:
                return _decode_value(arg, value)
            except Exception:
                continue
        return value
    if origin in (list, typing.List):
        (arg,) = typing.get_args(tp) or (typing.Any,)
        return [_decode_value(arg, v) for v in value]
    if origin in (dict, typing.Dict):
        args = typing.get_args(tp) or (typing.Any, typing.Any)
        return {k: _decode_value(args[1], v) for k, v in value.items()}
    if isinstance(tp, type) and dataclasses.is_dataclass(tp) and isinstance(value, dict):
        return decode(tp, value)
    if isinstance(tp, type) and issubclass(tp, enum.Enum) and not isinstance(value, tp):
        return tp(value)
    return value


def decode(cls, data):
    if isinstance(cls, type) and issubclass(cls, Registrable) and isinstance(data, dict) and "type" in data:
        data = dict(data)
        cls = cls.get_registered_class(data.pop("type"))
    hints = typing.get_type_hints(cls)
    kwargs = {}
    for f in dataclasses.fields(cls):
        if f.name in data and f.init:
            kwargs[f.name] = _decode_value(hints.get(f.name, typing.Any), data[f.name])
    return cls(**kwargs)
