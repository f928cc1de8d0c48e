"""B200 (sm_100a) AWQ W4A16 decode path of the Qwen3-8B-shape decoder.

The directory name is not a Python identifier; load it with
importlib.util.spec_from_file_location("qw3awq_b200", "<dir>/__init__.py", submodule_search_locations=["<dir>"]).

cabi  -- ctypes binding of libqw3awq.so (the C ABI of include/qw3_cabi.h)
infer -- QWen3AWQInfer, the reference's class (Inference.cu:356-366) over that ABI
ops   -- the per-operator entry points on torch device tensors (tests, bench)
"""
from . import cabi  # noqa: F401
from .infer import QWen3AWQInfer  # noqa: F401
