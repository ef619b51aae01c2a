"""Stand-in for `bettermap`: ordered map over a thread pool."""

from concurrent.futures import ThreadPoolExecutor


def ordered_map_per_thread(fn, seq, parallelism=None, **kwargs):
    with ThreadPoolExecutor(max_workers=parallelism or 4) as pool:
        yield from pool.map(fn, seq)


def map_per_process(fn, seq, **kwargs):
    return map(fn, seq)
