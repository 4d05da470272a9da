"""Global FLOP tally the kernels' Python wrappers feed while a profiler is active."""
_enabled = False
_total = 0
_listeners = []


def enabled() -> bool:
    return _enabled


def add(flops: int):
    global _total
    if _enabled:
        _total += int(flops)
        for fn in _listeners:
            fn(int(flops))


def start(listener=None):
    global _enabled, _total
    _enabled, _total = True, 0
    if listener is not None:
        _listeners.append(listener)


def stop() -> int:
    global _enabled
    _enabled = False
    _listeners.clear()
    return _total
