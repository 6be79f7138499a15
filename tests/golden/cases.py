"""Shapes of the small decode fixtures (shared by make_golden.py and the tests)."""
from oracle.ref_decode import Dims

SMALL_MOE = Dims(name="small_moe", H=512, NH=8, NKV=2, HD=128, INTER=0, L=2, V=1024, eps=1e-6, theta=1e6,
                 qk_norm=True, moe=True, E=16, TOPK=4, MI=128, norm_topk=True)
SMALL_DENSE = Dims(name="small_dense", H=256, NH=4, NKV=2, HD=64, INTER=640, L=2, V=512, eps=1e-6, theta=1e4,
                   tie=True, bias=True, qk_norm=False, moe=False)

# a small absorbed-MLA layer (DeepSeek-V2 family) for the MLA oracle fixture: keyword arguments of oracle.ref_mla.MlaDims
MLA_SMALL = dict(hidden=256, heads=4, kv_lora=64, qk_nope=32, qk_rope=16, v_head=32, moe_inter=48, n_routed=8, top_k=3, n_shared=2)
