"""Shapes of the small decode fixtures (shared by make_golden.py and the tests)."""
from oracle.ref_decode import Dims

SMALL_MOE = Dims(name="small_moe", H=512, NH=8, NKV=2, HD=128, INTER=0, L=2, V=1024, eps=1e-6, theta=1e6,
                 qk_norm=True, moe=True, E=16, TOPK=4, MI=128, norm_topk=True)
SMALL_DENSE = Dims(name="small_dense", H=256, NH=4, NKV=2, HD=64, INTER=640, L=2, V=512, eps=1e-6, theta=1e4,
                   tie=True, bias=True, qk_norm=False, moe=False)
