"""
Configuration system: ``Config`` dataclasses, a name->class ``Registrable`` registry, a typed
dict->dataclass decoder, dot-list overrides and the ``DType`` enum.

It offers the API of the reference's ``Config`` (src/olmo_core/config.py:55-405) without depending on
the external ``dataclass_extensions`` package: ``Registrable`` and ``decode`` are implemented here.
Dumped configs carry a ``_CLASS_`` field with the fully-qualified class name; names that start with
``olmo_core.`` (configs written by the reference) are resolved inside this package.
"""

from __future__ import annotations

import copy as _copy
import dataclasses
import importlib
import json
import typing
from dataclasses import dataclass, fields, is_dataclass
from enum import Enum
from typing import (
    Any,
    Callable,
    ClassVar,
    Dict,
    Generator,
    List,
    Optional,
    Sequence,
    Tuple,
    Type,
    TypeVar,
    Union,
)

import torch
import yaml

from .aliases import PathOrStr
from .exceptions import OLMoConfigurationError

__all__ = ["Config", "DType", "StrEnum", "UNSET", "Registrable", "decode", "encode"]

PACKAGE = __name__.split(".")[0]
_REFERENCE_PACKAGE = "olmo_core"


class StrEnum(str, Enum):
    """String-valued enum whose ``str()`` is its value."""

    def __str__(self) -> str:
        return self.value

    def __repr__(self) -> str:
        return f"'{str(self)}'"


# ----------------------------------------------------------------------------------------------
# Registrable
# ----------------------------------------------------------------------------------------------

R = TypeVar("R", bound="Registrable")


class Registrable:
    """
    Base for polymorphic configs. A direct subclass of ``Registrable`` owns a registry; its
    subclasses join it with ``@Base.register("name")``. The registered name is stored under ``"type"``
    when a config is dumped and selects the class when it is decoded.
    """

    _registry: ClassVar[Dict[type, Dict[str, type]]] = {}
    _default_type: ClassVar[Optional[str]] = None

    @classmethod
    def _registry_root(cls) -> type:
        root = cls
        for klass in cls.__mro__:
            if klass is Registrable:
                break
            if Registrable in klass.__bases__:
                root = klass
        return root

    @classmethod
    def register(cls, name: str, default: bool = False, exist_ok: bool = True) -> Callable[[Type[R]], Type[R]]:
        root = cls._registry_root()

        def deco(subclass: Type[R]) -> Type[R]:
            reg = Registrable._registry.setdefault(root, {})
            if name in reg and reg[name] is not subclass and not exist_ok:
                raise OLMoConfigurationError(f"'{name}' is already registered for {root.__name__}")
            reg[name] = subclass
            subclass._registered_name = name  # type: ignore[attr-defined]
            if default:
                root._default_type = name  # type: ignore[attr-defined]
            return subclass

        return deco

    @classmethod
    def get_registered_class(cls, name: str) -> type:
        root = cls._registry_root()
        reg = Registrable._registry.get(root, {})
        if name not in reg:
            raise OLMoConfigurationError(
                f"'{name}' is not a registered {root.__name__}; known: {sorted(reg)}"
            )
        return reg[name]

    @classmethod
    def get_registered_name(cls, sub: Optional[type] = None) -> Optional[str]:
        """Name under which ``sub`` (default: this class) was registered, or ``None``."""
        klass = sub or cls
        return klass.__dict__.get("_registered_name")

    @classmethod
    def get_registered_names(cls) -> List[str]:
        return sorted(Registrable._registry.get(cls._registry_root(), {}))


# ----------------------------------------------------------------------------------------------
# typed decoding
# ----------------------------------------------------------------------------------------------


def _resolve_class(name: str) -> Optional[type]:
    if "." not in name:
        return None
    module_name, _, cls_name = name.rpartition(".")
    candidates = [module_name]
    if module_name == _REFERENCE_PACKAGE or module_name.startswith(_REFERENCE_PACKAGE + "."):
        candidates.insert(0, PACKAGE + module_name[len(_REFERENCE_PACKAGE):])
    for mod in candidates:
        try:
            module = importlib.import_module(mod)
        except Exception:
            continue
        obj = module
        try:
            for part in cls_name.split("."):
                obj = getattr(obj, part)
        except AttributeError:
            continue
        if isinstance(obj, type):
            return obj
    return None


def _type_hints(cls: type) -> Dict[str, Any]:
    try:
        return typing.get_type_hints(cls)
    except Exception:
        return {f.name: f.type for f in fields(cls)}


def _is_optional(tp: Any) -> bool:
    return typing.get_origin(tp) is Union and type(None) in typing.get_args(tp)


def decode(tp: Any, value: Any, path: str = "") -> Any:
    """
    Coerce ``value`` (plain dicts / lists / scalars, e.g. parsed YAML) into the type ``tp``: dataclasses
    (honouring ``_CLASS_`` and ``type`` discriminators), ``Optional``/``Union``, enums, tuples, lists,
    dicts (digit-string keys become ints when the key type is ``int``), ``torch.dtype`` and scalars.
    """
    if tp is Any or tp is None or isinstance(tp, TypeVar):
        return _decode_untyped(value)
    if isinstance(tp, str):
        return _decode_untyped(value)
    origin = typing.get_origin(tp)
    args = typing.get_args(tp)

    if origin is Union or (origin is not None and str(origin) == "types.UnionType"):
        if value is None and type(None) in args:
            return None
        errors = []
        non_none = [a for a in args if a is not type(None)]
        # Prefer dataclass targets when the value is a mapping, scalars otherwise.
        ordered = sorted(non_none, key=lambda a: 0 if (isinstance(value, dict) == _is_dataclass_type(a)) else 1)
        for arg in ordered:
            try:
                return decode(arg, value, path)
            except (OLMoConfigurationError, TypeError, ValueError, KeyError) as e:
                errors.append(e)
        raise OLMoConfigurationError(f"cannot decode {value!r} at '{path}' as {tp}: {errors}")

    if _is_dataclass_type(tp) or (isinstance(value, dict) and "_CLASS_" in value):
        if is_dataclass(value) and not isinstance(value, type):
            return value
        if value is None:
            return None
        if not isinstance(value, dict):
            raise OLMoConfigurationError(f"expected a mapping for {tp} at '{path}', got {type(value).__name__}")
        return _decode_dataclass(tp, value, path)

    if origin in (list, typing.List, Sequence, typing.Sequence) or tp in (list, List):
        if value is None:
            return None
        (elem,) = args if args else (Any,)
        return [decode(elem, v, f"{path}.{i}") for i, v in enumerate(value)]
    if origin in (tuple, typing.Tuple) or tp is tuple:
        if value is None:
            return None
        if not args:
            return tuple(_decode_untyped(v) for v in value)
        if len(args) == 2 and args[1] is Ellipsis:
            return tuple(decode(args[0], v, f"{path}.{i}") for i, v in enumerate(value))
        return tuple(decode(a, v, f"{path}.{i}") for i, (a, v) in enumerate(zip(args, value)))
    if origin in (dict, typing.Dict) or tp is dict:
        if value is None:
            return None
        kt, vt = args if args else (Any, Any)
        out = {}
        for k, v in value.items():
            if kt is int and isinstance(k, str) and k.lstrip("-").isdigit():
                k = int(k)
            elif isinstance(k, str) and k.isdigit() and kt is Any:
                k = int(k)
            out[k] = decode(vt, v, f"{path}.{k}")
        return out
    if origin in (set, frozenset):
        return origin(decode(args[0] if args else Any, v, path) for v in value)
    if origin is typing.Literal:
        return value
    if origin is type or origin is typing.Type:
        return value
    if isinstance(tp, type):
        if value is None:
            return None
        if issubclass(tp, Enum):
            if isinstance(value, tp):
                return value
            try:
                return tp(value)
            except ValueError:
                try:
                    return tp[value]
                except KeyError:
                    raise OLMoConfigurationError(f"'{value}' is not a valid {tp.__name__} at '{path}'")
        if tp is torch.dtype:
            return value if isinstance(value, torch.dtype) else DType(str(value).replace("torch.", "")).as_pt()
        if tp is bool:
            if isinstance(value, str):
                return value.lower() in ("1", "true", "yes")
            return bool(value)
        if tp is float and isinstance(value, (int, float, str)):
            return float(value)
        if tp is int and isinstance(value, (int, str)) and not isinstance(value, bool):
            return int(value)
        if tp is int and isinstance(value, float) and value.is_integer():
            return int(value)
        if tp is str:
            return str(value)
        if isinstance(value, tp):
            return value
        if tp in (int, float) or isinstance(value, (dict, list)):
            raise OLMoConfigurationError(f"cannot decode {value!r} at '{path}' as {tp.__name__}")
    return _decode_untyped(value)


def _is_dataclass_type(tp: Any) -> bool:
    return isinstance(tp, type) and is_dataclass(tp)


def _decode_untyped(value: Any) -> Any:
    if isinstance(value, dict):
        if "_CLASS_" in value:
            return _decode_dataclass(None, value, "")
        return {(int(k) if isinstance(k, str) and k.isdigit() else k): _decode_untyped(v) for k, v in value.items()}
    if isinstance(value, list):
        return [_decode_untyped(v) for v in value]
    return value


def _decode_dataclass(tp: Optional[type], data: Dict[str, Any], path: str) -> Any:
    data = dict(data)
    cls: Optional[type] = tp if _is_dataclass_type(tp) else None
    cls_name = data.pop("_CLASS_", None)
    if cls_name is not None:
        resolved = _resolve_class(cls_name)
        if resolved is not None and (cls is None or issubclass(resolved, cls) or not issubclass(cls, resolved)):
            cls = resolved
    type_name = data.get("type")
    if cls is not None and isinstance(type_name, str) and issubclass(cls, Registrable):
        field_names = {f.name for f in fields(cls)}
        if cls_name is not None:
            if "type" not in field_names:
                data.pop("type")
        else:
            try:
                cls = cls.get_registered_class(type_name)
                if "type" not in {f.name for f in fields(cls)}:
                    data.pop("type")
            except OLMoConfigurationError:
                if "type" not in field_names:
                    raise
    elif cls is not None and cls_name is None and issubclass(cls, Registrable) and cls._default_type is not None:
        if dataclasses.is_dataclass(cls) and getattr(cls, "__abstractmethods__", None):
            cls = cls.get_registered_class(cls._default_type)
    if cls is None:
        raise OLMoConfigurationError(f"cannot determine the class of the mapping at '{path}'")
    for ignored in getattr(cls, "_IGNORE_FIELDS", ()):  # fields dropped from old configs
        data.pop(ignored, None)
    hints = _type_hints(cls)
    kwargs = {}
    init_fields = {f.name: f for f in fields(cls) if f.init}
    for fname, f in getattr(cls, "__dataclass_fields__", {}).items():
        if fname not in init_fields and "INITVAR" in str(getattr(f, "_field_type", "")):
            init_fields[fname] = f
    for key, val in data.items():
        if key not in init_fields:
            raise OLMoConfigurationError(f"'{cls.__name__}' has no field '{key}' (at '{path}')")
        kwargs[key] = decode(hints.get(key, Any), val, f"{path}.{key}" if path else key)
    try:
        return cls(**kwargs)
    except TypeError as e:
        raise OLMoConfigurationError(f"invalid arguments for {cls.__name__} at '{path}': {e}") from e


def encode(obj: Any) -> Any:
    """JSON-safe representation of configs, enums, dtypes, tuples and paths."""
    if isinstance(obj, Config):
        return obj.as_config_dict()
    if is_dataclass(obj) and not isinstance(obj, type):
        return {f.name: encode(getattr(obj, f.name)) for f in fields(obj)}
    if isinstance(obj, Enum):
        return obj.value
    if isinstance(obj, torch.dtype):
        return str(obj).replace("torch.", "")
    if isinstance(obj, dict):
        return {str(k) if not isinstance(k, (str, int, float, bool)) else k: encode(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple, set, frozenset)):
        return [encode(v) for v in obj]
    if isinstance(obj, (str, int, float, bool)) or obj is None:
        return obj
    return str(obj)


# ----------------------------------------------------------------------------------------------
# Config
# ----------------------------------------------------------------------------------------------

C = TypeVar("C", bound="Config")


@dataclass
class Config:
    """
    Base class for configuration dataclasses (subclasses are decorated with ``@dataclass`` too).
    """

    CLASS_NAME_FIELD: ClassVar[str] = "_CLASS_"

    def as_dict(
        self,
        *,
        exclude_none: bool = False,
        exclude_private_fields: bool = False,
        exclude: Optional[Iterable[str]] = None,
        include_class_name: bool = False,
        include_registered_name: bool = False,
        json_safe: bool = False,
        recurse: bool = True,
    ) -> Dict[str, Any]:
        """
        Convert to a dictionary (options of src/olmo_core/config.py:84-151). ``exclude`` drops fields by name at every
        level; ``include_class_name`` injects ``_CLASS_``; the registered ``type`` name of :class:`Registrable` configs is
        added with ``include_registered_name`` (and alongside the class name); ``json_safe`` converts enums, dtypes and
        tuples; ``recurse=False`` keeps nested configs as objects (the form builders pass to constructors). Fields that
        are not constructor arguments are left out.
        """
        excluded = set(exclude) if exclude is not None else set()

        def iter_fields(d) -> Generator[Tuple[str, Any], None, None]:
            for f in fields(d):
                if f.name in excluded or not f.init:
                    continue
                value = getattr(d, f.name)
                if exclude_none and value is None:
                    continue
                if exclude_private_fields and f.name.startswith("_"):
                    continue
                yield f.name, value

        def convert(d: Any, rec: bool = True) -> Any:
            if is_dataclass(d) and not isinstance(d, type):
                if not rec:
                    return d
                out = {k: convert(v) for k, v in iter_fields(d)}
                if include_class_name:
                    out[Config.CLASS_NAME_FIELD] = f"{d.__class__.__module__}.{d.__class__.__qualname__}"
                if (include_class_name or include_registered_name) and isinstance(d, Registrable) and "type" not in out:
                    name = d.get_registered_name(type(d))
                    if name is not None:
                        out["type"] = name
                return out
            if isinstance(d, dict):
                return {(encode(k) if json_safe else k): convert(v) for k, v in d.items()}
            if isinstance(d, (list, tuple, set)):
                seq = [convert(v) for v in d]
                if json_safe or isinstance(d, list):
                    return seq
                return type(d)(seq)
            if json_safe:
                return encode(d)
            return d

        if not recurse:
            return {k: v for k, v in iter_fields(self)}
        return convert(self)

    def as_config_dict(self) -> Dict[str, Any]:
        """JSON-safe dict that :meth:`from_dict` can rebuild the exact classes from."""
        return self.as_dict(exclude_none=True, exclude_private_fields=True, include_class_name=True,
                            include_registered_name=True, json_safe=True)

    def apply(self, func: Callable[["Config"], None]) -> None:
        """Call ``func`` on this config and, recursively, every config nested inside it."""

        def visit(d: Any) -> None:
            if isinstance(d, Config):
                func(d)
            if is_dataclass(d) and not isinstance(d, type):
                for f in fields(d):
                    visit(getattr(d, f.name))
            elif isinstance(d, dict):
                for v in d.values():
                    visit(v)
            elif isinstance(d, (list, tuple, set)):
                for v in d:
                    visit(v)

        visit(self)

    def validate(self) -> None:
        """Hook for subclasses; raises :class:`OLMoConfigurationError` on invalid settings."""

    def merge(self: C, dotlist: List[str], prefix: Optional[str] = None, strict: bool = True) -> C:
        """
        New config with ``--a.b=c`` style overrides applied. With ``prefix`` only options under that
        prefix are used. Values are parsed as YAML. ``strict=False`` skips keys that do not exist.
        """
        opts = _clean_opts(dotlist)
        if prefix is not None:
            pfx = prefix.rstrip(".") + "."
            opts = [(k[len(pfx):], v) for k, v in opts if k.startswith(pfx)]
        if not opts:
            return self
        data = self.as_dict(include_class_name=True)
        for key, value in opts:
            try:
                _set_nested(data, key, value)
            except (KeyError, IndexError, TypeError) as e:
                if strict:
                    raise OLMoConfigurationError(f"failed to apply override '{key}': {e}") from e
        try:
            return self.from_dict(data)
        except OLMoConfigurationError:
            if strict:
                raise
            return self

    def replace(self: C, **changes) -> C:
        return dataclasses.replace(self, **changes)

    def copy(self: C, deep: bool = True) -> C:
        return _copy.deepcopy(self) if deep else _copy.copy(self)

    @classmethod
    def from_dict(cls: Type[C], data: Dict[str, Any], overrides: Optional[List[str]] = None) -> C:
        data = _copy.deepcopy(data)
        if overrides:
            for key, value in _clean_opts(overrides):
                _set_nested(data, key, value)
        out = decode(cls, data)
        if not isinstance(out, cls):
            raise OLMoConfigurationError(f"decoded a {type(out).__name__}, expected {cls.__name__}")
        return out

    @classmethod
    def from_file(cls: Type[C], path: PathOrStr, overrides: Optional[List[str]] = None) -> C:
        p = str(path)
        if p.endswith((".yaml", ".yml")):
            return cls.from_yaml(path, overrides)
        return cls.from_json(path, overrides)

    @classmethod
    def from_json(cls: Type[C], path: PathOrStr, overrides: Optional[List[str]] = None) -> C:
        from .io import read_text

        return cls.from_dict(json.loads(read_text(path)), overrides)

    @classmethod
    def from_yaml(cls: Type[C], path: PathOrStr, overrides: Optional[List[str]] = None) -> C:
        from .io import read_text

        return cls.from_dict(yaml.safe_load(read_text(path)), overrides)


def _set_nested(data: Any, key: str, value: Any) -> None:
    parts = key.split(".")
    cur = data
    for i, part in enumerate(parts):
        last = i == len(parts) - 1
        if isinstance(cur, (list, tuple)):
            idx = int(part)
            if last:
                cur[idx] = value  # type: ignore[index]
            else:
                cur = cur[idx]
        elif isinstance(cur, dict):
            lookup: Any = part
            if part not in cur and part.isdigit() and int(part) in cur:
                lookup = int(part)
            if last:
                if isinstance(value, dict) and isinstance(cur.get(lookup), dict) and "_CLASS_" not in value:
                    # whole-dict override keeps the class unless the type discriminator changes
                    merged = dict(cur[lookup]) if "type" not in value else {}
                    merged.update(value)
                    cur[lookup] = merged
                else:
                    cur[lookup] = value
            else:
                if lookup not in cur or cur[lookup] is None:
                    raise KeyError(f"'{'.'.join(parts[: i + 1])}' does not exist")
                cur = cur[lookup]
        else:
            raise TypeError(f"cannot descend into {type(cur).__name__} at '{'.'.join(parts[:i])}'")


def _clean_opts(opts: Sequence[str]) -> List[Tuple[str, Any]]:
    return [_clean_opt(o) for o in opts]


def _clean_opt(arg: str) -> Tuple[str, Any]:
    if "=" not in arg:
        name, val = arg, "true"
    else:
        name, val = arg.split("=", 1)
    name = name.strip("-").replace("-", "_")
    return name, yaml.safe_load(val)


class DType(StrEnum):
    """String names of the supported ``torch.dtype`` values."""

    float32 = "float32"
    bfloat16 = "bfloat16"
    float16 = "float16"
    float64 = "float64"
    float8_e4m3fn = "float8_e4m3fn"
    float8_e5m2 = "float8_e5m2"

    @classmethod
    def from_pt(cls, dtype: torch.dtype) -> "DType":
        name = str(dtype).replace("torch.", "")
        try:
            return cls(name)
        except ValueError:
            raise NotImplementedError(dtype)

    def as_pt(self) -> torch.dtype:
        return getattr(torch, self.value)


class _Unset:
    """Sentinel for "argument not given" where ``None`` is a meaningful value."""

    _instance: ClassVar[Optional["_Unset"]] = None

    def __new__(cls):
        if cls._instance is None:
            cls._instance = super().__new__(cls)
        return cls._instance

    def __repr__(self) -> str:
        return "UNSET"

    def __bool__(self) -> bool:
        return False


UNSET: Any = _Unset()
