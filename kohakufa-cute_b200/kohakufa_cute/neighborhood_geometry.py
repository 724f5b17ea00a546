"""Integer geometry of the shifted neighbourhood window (host mirror of the device functions).

Forward: a query at coordinate ``p`` on an axis of extent ``e`` with window ``w`` sees keys
``[start, start + w)`` with ``start = clamp(p - w // 2, 0, e - w)``.  The relation is not symmetric
at the borders, so the key/value gradients enumerate the inverse set: the queries whose window
contains a key form the inclusive range returned by ``inverse_range``.
(Reference: src/kohakufa_cute/neighborhood_geometry.py:9-25 and neighborhood_kernels.py:193-212
of the reference project.)
"""


def window_start(position, extent, window):
    return min(max(position - window // 2, 0), extent - window)


def inverse_range(key, extent, window):
    """Inclusive (lo, hi) of query coordinates on this axis whose window holds ``key``."""
    lo = 0 if key - window + 1 <= 0 else key - window + 1 + window // 2
    hi = extent - 1 if key >= extent - window else key + window // 2
    return lo, hi
