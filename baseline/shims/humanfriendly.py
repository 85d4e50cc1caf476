"""Stand-in for the absent ``humanfriendly`` package: the two functions the reference calls."""
import re

_UNITS = {'b': 1, 'byte': 1, 'bytes': 1,
          'kb': 1000, 'mb': 1000 ** 2, 'gb': 1000 ** 3, 'tb': 1000 ** 4,
          'kib': 1024, 'mib': 1024 ** 2, 'gib': 1024 ** 3, 'tib': 1024 ** 4,
          'k': 1000, 'm': 1000 ** 2, 'g': 1000 ** 3, 't': 1000 ** 4}


def parse_size(text, binary=False):
    m = re.fullmatch(r'\s*([0-9]*\.?[0-9]+)\s*([A-Za-z]*)\s*', str(text))
    if not m:
        raise ValueError(f'cannot parse size {text!r}')
    unit = m.group(2).lower()
    if unit == '':
        return int(float(m.group(1)))
    mult = _UNITS[unit]
    if binary and unit in ('kb', 'mb', 'gb', 'tb', 'k', 'm', 'g', 't'):
        mult = 1024 ** ('kmgt'.index(unit[0]) + 1)
    return int(float(m.group(1)) * mult)


def format_size(num_bytes, keep_width=False, binary=False):
    base = 1024 if binary else 1000
    names = ['bytes', 'KiB', 'MiB', 'GiB', 'TiB'] if binary else ['bytes', 'KB', 'MB', 'GB', 'TB']
    if num_bytes < base:
        return f'{int(num_bytes)} byte' + ('' if num_bytes == 1 else 's')
    value = float(num_bytes)
    for name in names[1:]:
        value /= base
        if value < base or name == names[-1]:
            text = f'{value:.2f}'.rstrip('0').rstrip('.')
            return f'{text} {name}'
