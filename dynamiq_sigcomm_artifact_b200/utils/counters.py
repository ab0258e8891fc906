"""Count launches of this package's own kernels (reported by bench.py as ``gpu_launches``)."""
from collections import Counter

LAUNCHES: Counter = Counter()


def add(name: str, n: int = 1) -> None:
    LAUNCHES[name] += n


def total() -> int:
    return sum(LAUNCHES.values())


def reset() -> None:
    LAUNCHES.clear()
