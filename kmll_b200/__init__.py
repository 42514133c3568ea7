"""kmll_b200 — B200 (sm_100a) implementation of kmll's quantized decode path.

`ops` mirrors kmll's operator API over the C ABI of libkmll_b200.so; `runtime` drives whole-model
decode through the C++ runtime inside the same library.  The library is built in-tree by
`python -m kmll_b200.build`; there is no CPU fallback.
"""
from .lib import KmllError, load  # noqa: F401

__all__ = ["KmllError", "load"]
