"""Human-readable byte sizes ("1MB", "82.94 KB", "4 GiB").

The reference delegates to the third-party ``humanfriendly`` package
(``msccl/autosynth/registry.py:22-32``, ``msccl/autosynth/__init__.py:119-123``); these two
functions reproduce the behaviour relied on there: decimal units for KB/MB/GB, binary for
KiB/MiB/GiB, at most two decimals when formatting.
"""
import re

_DECIMAL = {'': 1, 'b': 1, 'byte': 1, 'bytes': 1, 'k': 10 ** 3, 'kb': 10 ** 3, 'm': 10 ** 6, 'mb': 10 ** 6,
            'g': 10 ** 9, 'gb': 10 ** 9, 't': 10 ** 12, 'tb': 10 ** 12, 'p': 10 ** 15, 'pb': 10 ** 15}
_BINARY = {'kib': 2 ** 10, 'mib': 2 ** 20, 'gib': 2 ** 30, 'tib': 2 ** 40, 'pib': 2 ** 50}
_PATTERN = re.compile(r'^\s*([0-9]+(?:\.[0-9]+)?|\.[0-9]+)\s*([A-Za-z]*)\s*$')


def parse_size(text):
    """'512B' -> 512, '1MB' -> 1000000, '1GiB' -> 1073741824; ints pass through."""
    if isinstance(text, (int, float)):
        return int(text)
    m = _PATTERN.match(text)
    if not m:
        raise ValueError(f'Failed to parse size! (input {text!r})')
    unit = m.group(2).lower()
    scale = _DECIMAL.get(unit, _BINARY.get(unit))
    if scale is None:
        raise ValueError(f'Failed to parse size! (input {text!r} has unknown unit {m.group(2)!r})')
    return int(float(m.group(1)) * scale)


def format_size(num_bytes):
    """82944 -> '82.94 KB', 512 -> '512 bytes', 1 -> '1 byte'."""
    if num_bytes < 1000:
        n = int(num_bytes)
        return f'{n} byte' if n == 1 else f'{n} bytes'
    value = float(num_bytes)
    for unit in ('KB', 'MB', 'GB', 'TB', 'PB'):
        value /= 1000
        if value < 1000 or unit == 'PB':
            text = f'{value:.2f}'.rstrip('0').rstrip('.')
            return f'{text} {unit}'
