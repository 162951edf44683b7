"""Helpers of the communicator; mirrors the used part of
``chainerkfac/communicators/_utility.py`` (``get_nelems`` :72-83)."""


def get_nelems(arrays):
    """Wire elements of nested ``arrays[rank] = [(array, triangular), ...]``."""
    nelems = 0
    for local_arrays in arrays:
        nelems += get_local_nelems(local_arrays)
    return nelems


def get_local_nelems(local_arrays):
    nelems = 0
    for array, triangular in local_arrays:
        if triangular:
            if array.shape[0] != array.shape[1]:
                raise RuntimeError('get_nelems: not a square matrix')
            nelems += array.shape[0] * (array.shape[0] + 1) // 2
        else:
            nelems += array.numel() if hasattr(array, 'numel') else array.size
    return nelems


def wire_torch_dtype(name):
    """torch dtype of a wire element type given by name (or dtype)."""
    import torch
    table = {'float32': torch.float32, 'float16': torch.float16,
             'bfloat16': torch.bfloat16}
    if isinstance(name, torch.dtype):
        name = str(name).replace('torch.', '')
    if name not in table:
        raise ValueError('wire_dtype must be one of {}, not {}'.format(
            sorted(table), name))
    return table[name]
