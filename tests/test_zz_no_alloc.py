"""The attention entry point that allocates nothing (etxb_attn_fused_static) against the regular fused-attention tile.

Who needs it: callers that must not, or cannot, allocate device memory when they run attention -- a plug-in that is
only handed its host's input and output buffers, a serving loop whose pools were sized once at start-up, a process
that already gave all free HBM to its KV cache.  The regular tile takes its partial-result scratch from the caller;
this entry keeps it in a fixed static device array inside the library (limits: NH <= 64, 64 partitions of 32
positions, head_dim <= 128).  The outputs must be identical to the regular entry's, on two calls in a row (the array
keeps the previous call's contents, so the second call checks that what must start at zero is cleared).

Collected last on purpose (file name): a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import etx_megakernel_b200  # noqa: E402,F401
from etx_megakernel_b200 import ops  # noqa: E402
from etx_megakernel_b200.importer import argblock  # noqa: E402
from etx_megakernel_b200.models import qwen as Q  # noqa: E402
from etx_megakernel_b200.runtime import EtxbError, attn_fused_static, op_launch  # noqa: E402

DEV = "cuda:0"
ENT = ops.all_entries()


def _case(NH, NKV, HD, seq, seed):
    g = torch.Generator(device=DEV); g.manual_seed(seed)
    maxlen = ((seq + 31) // 32) * 32 + 32
    nblk, parts = maxlen // 16, maxlen // 32
    t = {"qkv": torch.randn((NH + 2 * NKV, HD), device=DEV, generator=g).bfloat16(),
         "qn": (1 + 0.1 * torch.randn(HD, device=DEV, generator=g)).bfloat16(), "kn": (1 + 0.1 * torch.randn(HD, device=DEV, generator=g)).bfloat16(),
         "kc": (0.5 * torch.randn((nblk, NKV, HD // 8, 16, 8), device=DEV, generator=g)).bfloat16(),
         "vc": torch.randn((nblk, NKV, HD, 16), device=DEV, generator=g).bfloat16(),
         "cs": torch.from_numpy(Q.rope_table(1e6, HD, maxlen).view(np.int16)).to(DEV).view(torch.bfloat16),
         "bt": torch.arange(nblk, dtype=torch.int32, device=DEV), "sl": torch.tensor([seq], dtype=torch.int32, device=DEV),
         "pos": torch.tensor([seq - 1], dtype=torch.int64, device=DEV)}
    return t, parts


def _block(t, parts, NH, NKV, HD, kc, vc, out, scratch=None):
    s = scratch or {}
    return argblock.pack_named(ENT["attn_fused"], (parts * NKV, 1, 1), qkv=t["qkv"].data_ptr(), qw=t["qn"].data_ptr(), kw=t["kn"].data_ptr(),
                               cos_sin=t["cs"].data_ptr(), kc=kc.data_ptr(), vc=vc.data_ptr(), block_tables=t["bt"].data_ptr(),
                               seq_lens=t["sl"].data_ptr(), positions=t["pos"].data_ptr(), slot_mapping=t["pos"].data_ptr(),
                               exp_sums=s["es"].data_ptr() if s else 0, max_logits=s["ml"].data_ptr() if s else 0,
                               tmp_out=s["tmp"].data_ptr() if s else 0, out=out.data_ptr(), counters=s["cnt"].data_ptr() if s else 0,
                               scale=float(HD) ** -0.5, eps=1e-6, NH=NH, NKV=NKV, HD=HD, BS=16, X=8, max_parts=parts)


@pytest.mark.parametrize("NH,NKV,HD,seq", [(32, 4, 128, 1025), (8, 2, 128, 40)])
def test_static_scratch_entry_matches_regular_entry_twice(NH, NKV, HD, seq):
    outs = []
    for call in range(2):                                                 # two different inputs, one after the other
        t, parts = _case(NH, NKV, HD, seq, seed=call)
        kc_a, vc_a, kc_b, vc_b = t["kc"].clone(), t["vc"].clone(), t["kc"].clone(), t["vc"].clone()
        out_a = torch.zeros((NH, HD), dtype=torch.bfloat16, device=DEV); out_b = torch.zeros_like(out_a)
        scratch = {"es": torch.zeros((NH, parts), device=DEV), "ml": torch.zeros((NH, parts), device=DEV),
                   "tmp": torch.zeros((NH, parts, HD), device=DEV), "cnt": torch.zeros(NKV, dtype=torch.int32, device=DEV)}
        op_launch("attn_fused", _block(t, parts, NH, NKV, HD, kc_a, vc_a, out_a, scratch), parts * NKV)
        attn_fused_static(_block(t, parts, NH, NKV, HD, kc_b, vc_b, out_b))
        torch.cuda.synchronize()
        assert torch.equal(out_a, out_b), f"call {call}: outputs differ"   # same arithmetic: bit-identical, tolerance 0
        assert torch.equal(kc_a, kc_b) and torch.equal(vc_a, vc_b)
        assert float(out_b.float().abs().max()) > 0
        outs.append(out_b.clone())
    assert not torch.equal(outs[0], outs[1])                              # the two calls really had different inputs


def test_static_scratch_entry_rejects_sizes_beyond_its_array():
    t, parts = _case(8, 2, 128, 40, seed=0)
    out = torch.zeros((8, 128), dtype=torch.bfloat16, device=DEV)
    blk = bytearray(_block(t, parts, 8, 2, 128, t["kc"], t["vc"], out))
    import struct
    struct.pack_into("<i", blk, 148, 65)                                  # max_parts beyond the 64 the static array holds
    struct.pack_into("<IIII", blk, 160, 65 * 2, 1, 1, 65 * 2)
    with pytest.raises(EtxbError) as e:
        attn_fused_static(bytes(blk))
    assert e.value.status == "E_UNSUPPORTED" and "exceed the static scratch" in str(e.value)
