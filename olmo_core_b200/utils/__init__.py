"""
General helpers: device selection, seeding, rank-aware logging, CLI environment set-up, formatting,
stream registry, FLOP counting. Same function names as the reference's src/olmo_core/utils.py:41-847.
"""

from __future__ import annotations

import gc
import logging
import math
import os
import random
import socket
import sys
import threading
import time
import uuid
import warnings
from contextlib import contextmanager
from datetime import timedelta
from itertools import cycle, islice
from queue import Queue
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, TypeVar, Union

import numpy as np
import torch

from ..config import StrEnum
from ..exceptions import OLMoCLIError, OLMoEnvironmentError, OLMoError, OLMoThreadError

__all__ = [
    "LOG_FILTER_TYPE_ENV_VAR",
    "generate_uuid",
    "get_default_thread_count",
    "wait_for",
    "apply_to_tensors",
    "move_to_device",
    "mark_dynamic",
    "get_default_device",
    "has_compute_capability",
    "seed_all",
    "same_storage",
    "gc_cuda",
    "has_flash_attn",
    "set_env_var",
    "log_or_print",
    "LogFilterType",
    "log_extra_field",
    "setup_logging",
    "logging_configured",
    "excepthook",
    "install_excepthook",
    "filter_warnings",
    "set_env_variables",
    "prepare_cli_environment",
    "threaded_generator",
    "roundrobin",
    "powers_of_2",
    "capped_powers_of_2",
    "format_float",
    "format_int",
    "format_timedelta",
    "flatten_dict",
    "cuda_sync_debug_mode",
    "get_element_size",
    "ensure_multiple_of",
    "log_once",
    "warn_once",
    "info_value_of_dtype",
    "min_value_of_dtype",
    "get_or_init_stream",
    "record_flops",
]

log = logging.getLogger(__name__)
T = TypeVar("T")

_LOG_EXTRA_FIELDS: Dict[str, Any] = {}
_LOGGING_CONFIGURED = False


def generate_uuid() -> str:
    return str(uuid.uuid4())


def get_default_thread_count() -> int:
    env = os.environ.get("OLMO_NUM_THREADS_ENV_VAR") or os.environ.get("OLMO_NUM_THREADS")
    if env:
        return int(env)
    return min(16, (os.cpu_count() or 1) + 4)


def wait_for(condition: Callable[[], bool], description: str, timeout: float = 10.0) -> None:
    """Poll ``condition`` until it holds; raise ``TimeoutError`` after ``timeout`` seconds."""
    start = time.monotonic()
    while not condition():
        time.sleep(0.25)
        if time.monotonic() - start > timeout:
            raise TimeoutError(f"{description} timed out after {timeout:.0f}s")


def apply_to_tensors(fn: Callable[[torch.Tensor], None], container: Any) -> None:
    if isinstance(container, torch.Tensor):
        fn(container)
    elif isinstance(container, (list, tuple, set)):
        for x in container:
            apply_to_tensors(fn, x)
    elif isinstance(container, dict):
        for x in container.values():
            apply_to_tensors(fn, x)
    elif hasattr(container, "__dataclass_fields__"):
        for f in container.__dataclass_fields__:
            apply_to_tensors(fn, getattr(container, f))


def move_to_device(o: T, device: torch.device, non_blocking: Optional[bool] = None) -> T:
    """Move every tensor inside a nested container to ``device`` (non-blocking for CUDA targets)."""
    if non_blocking is None:
        non_blocking = device.type != "cpu"
    if isinstance(o, torch.Tensor):
        return o.to(device, non_blocking=non_blocking)  # type: ignore[return-value]
    if isinstance(o, dict):
        return {k: move_to_device(v, device, non_blocking) for k, v in o.items()}  # type: ignore[return-value]
    if isinstance(o, list):
        return [move_to_device(x, device, non_blocking) for x in o]  # type: ignore[return-value]
    if isinstance(o, tuple):
        return tuple(move_to_device(x, device, non_blocking) for x in o)  # type: ignore[return-value]
    return o


def mark_dynamic(x: torch.Tensor, dim: Union[int, Sequence[int]], strict: bool = True) -> None:
    """No tracing compiler is used on the GPU path, so shape annotations are a no-op."""


def get_default_device() -> torch.device:
    if torch.cuda.is_available() and torch.cuda.is_initialized():
        return torch.device("cuda")
    if torch.cuda.is_available() and "LOCAL_RANK" in os.environ:
        return torch.device("cuda")
    if torch.cuda.is_available():
        return torch.device("cuda")
    return torch.device("cpu")


def has_compute_capability(major: int, minor: int) -> bool:
    if not torch.cuda.is_available():
        return False
    return torch.cuda.get_device_capability() >= (major, minor)


def seed_all(seed: int) -> None:
    if seed < 0 or seed > 2**32 - 1:
        raise ValueError(f"seed {seed} is outside [0, 2^32 - 1]")
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def same_storage(x: torch.Tensor, y: torch.Tensor) -> bool:
    return x.untyped_storage().data_ptr() == y.untyped_storage().data_ptr()


def gc_cuda() -> None:
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def has_flash_attn() -> bool:
    """The GPU attention path is the in-tree kernel; no external flash-attn package is consulted."""
    return False


def set_env_var(name: str, value: str, override: bool = False, secret: bool = False) -> None:
    shown = "****" if secret else value
    if name in os.environ:
        if override and os.environ[name] != value:
            log_or_print(log, f"overriding env var '{name}' to '{shown}'")
            os.environ[name] = value
    else:
        log_or_print(log, f"setting env var '{name}' to '{shown}'")
        os.environ[name] = value


def log_or_print(logger: logging.Logger, msg: str, level: int = logging.INFO) -> None:
    if logging_configured():
        logger.log(level, msg)
    else:
        print(msg)


class LogFilterType(StrEnum):
    rank0_only = "rank0_only"
    local_rank0_only = "local_rank0_only"
    all_ranks = "all_ranks"


def log_extra_field(field_name: str, field_value: Any) -> None:
    """Attach a field to every subsequent log record (e.g. ``hostname``)."""
    _LOG_EXTRA_FIELDS[field_name] = field_value


def setup_logging(log_filter_type: LogFilterType = LogFilterType.rank0_only, force: bool = False) -> None:
    """Root logger with a rank-prefixed format and a filter that silences non-selected ranks below WARNING.
    A second call does nothing unless ``force`` is set."""
    global _LOGGING_CONFIGURED
    if _LOGGING_CONFIGURED and not force:
        return
    from ..distributed.utils import get_local_rank, get_rank

    log_extra_field("hostname", socket.gethostname())
    rank = get_rank() if "RANK" in os.environ or torch.distributed.is_initialized() else 0
    local_rank = get_local_rank() if "LOCAL_RANK" in os.environ else 0
    log_extra_field("global_rank", rank)
    log_extra_field("local_rank", local_rank)

    old_factory = logging.getLogRecordFactory()
    if not getattr(old_factory, "_ocb_wrapped", False):

        def factory(*args, **kwargs):
            record = old_factory(*args, **kwargs)
            for k, v in _LOG_EXTRA_FIELDS.items():
                setattr(record, k, v)
            return record

        factory._ocb_wrapped = True  # type: ignore[attr-defined]
        logging.setLogRecordFactory(factory)

    handler: logging.Handler = logging.StreamHandler(sys.stdout)
    handler.setFormatter(
        logging.Formatter(
            "%(asctime)s\t%(hostname)s:%(local_rank)s\t%(name)s:%(lineno)s\t%(levelname)s\t%(message)s",
            datefmt="%Y-%m-%d %H:%M:%S",
        )
    )

    def rank_filter(record: logging.LogRecord) -> int:
        if record.levelno > logging.INFO:
            return 1
        if log_filter_type == LogFilterType.all_ranks:
            return 1
        if log_filter_type == LogFilterType.rank0_only:
            return int(getattr(record, "global_rank", 0) == 0)
        return int(getattr(record, "local_rank", 0) == 0)

    handler.addFilter(rank_filter)
    logging.basicConfig(handlers=[handler], level=logging.INFO, force=True)
    logging.captureWarnings(True)
    logging.getLogger("urllib3").setLevel(logging.ERROR)
    _LOGGING_CONFIGURED = True


def logging_configured() -> bool:
    return _LOGGING_CONFIGURED or bool(logging.getLogger().handlers)


def excepthook(exctype, value, traceback) -> None:
    """Log uncaught exceptions (with the rank prefix) instead of printing a bare traceback."""
    if issubclass(exctype, KeyboardInterrupt):
        sys.__excepthook__(exctype, value, traceback)
    elif issubclass(exctype, OLMoCLIError):
        log.error(f"{exctype.__name__}: {value}")
    else:
        log.critical(f"Uncaught {exctype.__name__}: {value}", exc_info=(exctype, value, traceback))


def install_excepthook() -> None:
    sys.excepthook = excepthook


def filter_warnings() -> None:
    warnings.filterwarnings("ignore", category=UserWarning, message="torch.distributed.*_base is a private function.*")
    warnings.filterwarnings("ignore", category=UserWarning, message="TypedStorage is deprecated.*")
    warnings.filterwarnings("ignore", category=UserWarning, message="Please use DTensor instead.*")
    warnings.filterwarnings("ignore", category=FutureWarning, message="torch.distributed.checkpoint.*")
    warnings.filterwarnings("ignore", message=".*does not support reading from buffer.*")


def set_env_variables() -> None:
    os.environ.setdefault("OMP_NUM_THREADS", "8")
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")


LOG_FILTER_TYPE_ENV_VAR = "LOG_FILTER_TYPE"


def prepare_cli_environment(log_filter_type: Optional[LogFilterType] = None) -> None:
    """Logging, exception hook, warning filters and env vars for a command-line entry point."""
    if log_filter_type is None:
        log_filter_type = LogFilterType(os.environ.get(LOG_FILTER_TYPE_ENV_VAR, "rank0_only"))
    setup_logging(log_filter_type)
    install_excepthook()
    filter_warnings()
    set_env_variables()


def threaded_generator(g: Iterable[T], maxsize: int = 16, thread_name: Optional[str] = None):
    """Run generator ``g`` in a background thread, handing items over through a bounded queue."""
    q: Queue = Queue(maxsize=maxsize)
    sentinel = object()

    def fill() -> None:
        try:
            for item in g:
                q.put(item)
        except Exception as e:  # forwarded to the consumer
            q.put(e)
        finally:
            q.put(sentinel)

    thread = threading.Thread(name=thread_name, target=fill, daemon=True)
    thread.start()
    while True:
        item = q.get()
        if item is sentinel:
            break
        if isinstance(item, Exception):
            raise OLMoThreadError(f"generator thread {thread_name} failed") from item
        yield item
    thread.join()


def roundrobin(*iterables):
    """``roundrobin('ABC', 'D', 'EF') -> A D E B F C``"""
    active = len(iterables)
    nexts = cycle(iter(it).__next__ for it in iterables)
    while active:
        try:
            for nxt in nexts:
                yield nxt()
        except StopIteration:
            active -= 1
            nexts = cycle(islice(nexts, active))


def powers_of_2(x: int) -> List[int]:
    """Decompose ``x`` into its power-of-two summands, largest first."""
    out, bit = [], 1 << max(x.bit_length() - 1, 0)
    while bit:
        if x & bit:
            out.append(bit)
        bit >>= 1
    return out


def capped_powers_of_2(x: int, cap: int) -> List[int]:
    out: List[int] = []
    for p in powers_of_2(x):
        if p > cap:
            out.extend([cap] * (p // cap))
        else:
            out.append(p)
    return out


def format_float(value: float) -> str:
    if value == 0 or not math.isfinite(value):
        return f"{value}"
    mag = abs(value)
    if mag < 1e-4 or mag >= 1e9:
        return f"{value:.3E}"
    if mag < 1:
        return f"{value:.5f}".rstrip("0")
    if mag < 10:
        return f"{value:.3f}"
    if mag < 1000:
        return f"{value:.2f}" if mag < 100 else f"{value:.1f}"
    return f"{int(value):,d}"


def format_int(count: int) -> str:
    if count < 1_000:
        return str(count)
    if count < 1_000_000:
        return f"{count / 1_000:.1f}K".replace(".0K", "K")
    if count < 1_000_000_000:
        return f"{count / 1_000_000:.1f}M".replace(".0M", "M")
    if count < 1_000_000_000_000:
        return f"{count / 1_000_000_000:.1f}B".replace(".0B", "B")
    return f"{count / 1_000_000_000_000:.1f}T".replace(".0T", "T")


def format_timedelta(td: timedelta) -> str:
    total = int(td.total_seconds())
    days, rem = divmod(total, 86400)
    hours, rem = divmod(rem, 3600)
    minutes, seconds = divmod(rem, 60)
    parts = []
    if days:
        parts.append(f"{days}d")
    if hours:
        parts.append(f"{hours}h")
    if minutes:
        parts.append(f"{minutes}m")
    if seconds or not parts:
        parts.append(f"{seconds}s")
    return ", ".join(parts)


def flatten_dict(d: Dict[str, Any], sep: str = ".") -> Dict[str, Any]:
    out: Dict[str, Any] = {}

    def visit(prefix: str, sub: Dict[str, Any]) -> None:
        for k, v in sub.items():
            key = f"{prefix}{sep}{k}" if prefix else str(k)
            if isinstance(v, dict):
                visit(key, v)
            else:
                out[key] = v

    visit("", d)
    return out


@contextmanager
def cuda_sync_debug_mode(debug_mode: Union[int, str]):
    """Temporarily set ``torch.cuda.set_sync_debug_mode`` (surfaces accidental host-device syncs)."""
    current = None
    try:
        if torch.cuda.is_available():
            current = torch.cuda.get_sync_debug_mode()
            torch.cuda.set_sync_debug_mode(debug_mode)
        yield
    finally:
        if current is not None:
            torch.cuda.set_sync_debug_mode(current)


def get_element_size(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def ensure_multiple_of(x: int, of: int) -> int:
    return of * math.ceil(x / of)


_LOGGED: set = set()


def log_once(logger: logging.Logger, msg: str, *args, level: int = logging.INFO, **kwargs) -> None:
    if msg not in _LOGGED:
        _LOGGED.add(msg)
        logger.log(level, msg, *args, **kwargs)


def warn_once(msg: str, *args, **kwargs) -> None:
    if msg not in _LOGGED:
        _LOGGED.add(msg)
        warnings.warn(msg, *args, **kwargs)


def info_value_of_dtype(dtype: torch.dtype):
    if dtype == torch.bool:
        raise TypeError("bool has no numeric range")
    return torch.finfo(dtype) if dtype.is_floating_point else torch.iinfo(dtype)


def min_value_of_dtype(dtype: torch.dtype):
    return info_value_of_dtype(dtype).min


_STREAMS: Dict[str, "torch.cuda.Stream"] = {}


def get_or_init_stream(id: str, priority: int = 0) -> "torch.cuda.Stream":
    """Named side streams (e.g. ``"ag"``, ``"rs"``) created once per process."""
    key = f"{id}:{torch.cuda.current_device()}"
    if key not in _STREAMS:
        _STREAMS[key] = torch.cuda.Stream(priority=priority)
    return _STREAMS[key]


def record_flops(model: torch.nn.Module, *inputs, with_backward: bool = False, **kwargs) -> int:
    """Measured FLOPs of one forward (and backward) pass using ``FlopCounterMode``."""
    from torch.utils.flop_counter import FlopCounterMode

    with FlopCounterMode(display=False) as counter:
        out = model(*inputs, **kwargs)
        if with_backward:
            loss = out if isinstance(out, torch.Tensor) else out[0]
            loss.float().sum().backward()
    return counter.get_total_flops()
