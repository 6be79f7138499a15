"""CPU tests of the weight pack file (vl.bin / vl.manifest) and golden token file readers and writers."""
import numpy as np
import pytest

import etx_megakernel_b200  # noqa: F401
from etx_megakernel_b200.models import packfile as PF
from etx_megakernel_b200.models import qwen as Q
from oracle import ref_decode as O
from tests.golden.cases import SMALL_DENSE, SMALL_MOE


def _dims(od):
    return Q.Dims(**{f: getattr(od, f) for f in ("name", "H", "NH", "NKV", "HD", "INTER", "L", "V", "eps", "theta", "tie", "bias",
                                                 "qk_norm", "moe", "E", "TOPK", "MI", "norm_topk")})


@pytest.mark.parametrize("od", [SMALL_MOE, SMALL_DENSE], ids=["moe", "dense"])
def test_pack_file_round_trip_and_layout(tmp_path, od):
    d = _dims(od)
    packed = Q.pack_hf(d, O.SyntheticWeights(od, seed=4).get, 64)
    size = PF.write_vl(tmp_path, d, packed, 64)
    assert (tmp_path / "vl.bin").stat().st_size == size
    cfg, tens = PF.read_manifest(tmp_path / "vl.manifest")
    assert cfg["H"] == d.H and cfg["moe"] == int(d.moe) and cfg["bytes"] == size and abs(cfg["eps"] - d.eps) < 1e-12
    assert all(off % 256 == 0 for off, _ in tens.values())                       # every tensor on a 256-byte boundary
    assert list(tens)[:2] == ["embed", "final_norm"] and "L1.wqkv" in tens and ("L0.w13" in tens) == d.moe
    d2, maxlen, back = PF.read_vl(tmp_path, theta=d.theta)
    assert maxlen == 64 and (d2.H, d2.NH, d2.NKV, d2.HD, d2.L, d2.V, d2.moe, d2.E, d2.TOPK, d2.MI) == (d.H, d.NH, d.NKV, d.HD, d.L, d.V, d.moe, d.E, d.TOPK, d.MI)
    assert set(back) == set(packed)
    for k in packed:
        assert np.array_equal(back[k], packed[k]), k


def test_pack_file_reader_refuses_what_it_cannot_run(tmp_path):
    d = _dims(SMALL_DENSE)
    PF.write_vl(tmp_path, d, Q.pack_hf(d, O.SyntheticWeights(SMALL_DENSE, seed=4).get, 64), 64)
    man = tmp_path / "vl.manifest"
    text = man.read_text()
    man.write_text(text + "t L0.ln1b 0 256\n")                                    # a LayerNorm bias: a model kind without tiles here
    with pytest.raises(ValueError, match="no use for"):
        PF.read_vl(tmp_path)
    man.write_text(text.replace("cfg tie 1", "cfg tie 1\ncfg sparsemixer 1"))
    with pytest.raises(ValueError, match="sparsemixer"):
        PF.read_vl(tmp_path)
    man.write_text("\n".join(l for l in text.splitlines() if not l.startswith("t L1.wo ")) + "\n")
    with pytest.raises(ValueError, match="L1.wo is missing"):
        PF.read_vl(tmp_path)
    man.write_text(text.replace("cfg V ", "cfg V 1"))                             # a vocabulary the file does not hold
    with pytest.raises(ValueError, match="do not fit shape"):
        PF.read_vl(tmp_path)
    man.write_text(text + "bogus line\n")
    with pytest.raises(ValueError, match="not a manifest line"):
        PF.read_vl(tmp_path)


def test_golden_token_file_and_gate(tmp_path):
    p = tmp_path / "golden_c8.txt"
    PF.write_golden(p, [5, 6, 7], [10, 11, 12, 13], [2.5, 0.0001, 3.0, 1.0])
    assert p.read_text().splitlines()[0] == "prompt: 5 6 7" and p.read_text().splitlines()[2].startswith("margin: 2.5000 0.0001")
    prompt, gen, margins = PF.read_golden(p)
    assert (prompt, gen) == ([5, 6, 7], [10, 11, 12, 13]) and margins[1] == pytest.approx(1e-4)
    assert PF.check_golden([10, 11, 12, 13], gen, margins) == []
    assert PF.check_golden([10, 99, 1, 2], gen, margins, tie_margin=0.001) == []     # differs where the reference itself was at a tie
    assert "token 2" in PF.check_golden([10, 11, 99, 13], gen, margins, tie_margin=0.001)[0]
    assert "only 2 of 4" in PF.check_golden([10, 11], gen, margins)[0]
    (tmp_path / "bad.txt").write_text("prompt: 1\ngen: 2 3\nmargin: 1.0\n")
    with pytest.raises(ValueError, match="margins"):
        PF.read_golden(tmp_path / "bad.txt")
