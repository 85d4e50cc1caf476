from msccl.collectives import build_collective


def null_collective(n):
    return build_collective(f'Null(n={n})', n, 1, lambda r, c: True, lambda r, c: False)


def impossible_collective(n):
    return build_collective(f'Impossible(n={n})', n, 1, lambda r, c: False, lambda r, c: True)
