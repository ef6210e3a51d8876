"""Largest observed error per tolerance class over a test run.

The parity tests assert `error < tolerance`; they also call `note(name, error, tolerance)` so the
end-of-run summary (tests/conftest.py) shows how much of each tolerance the kernels actually used."""
WORST: dict[str, tuple[float, float, int]] = {}


def note(name: str, value: float, tol: float) -> float:
    value = float(value)
    cur = WORST.get(name)
    n = 1 if cur is None else cur[2] + 1
    if cur is None or value > cur[0]:
        WORST[name] = (value, float(tol), n)
    else:
        WORST[name] = (cur[0], cur[1], n)
    return value
