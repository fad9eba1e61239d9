import collections.abc
from itertools import repeat

from torch.nn.init import trunc_normal_  # noqa: F401  (same algorithm and argument order as timm's)


def _ntuple(n):
    def parse(x):
        if isinstance(x, collections.abc.Iterable) and not isinstance(x, str):
            return tuple(x)
        return tuple(repeat(x, n))
    return parse


to_2tuple = _ntuple(2)
