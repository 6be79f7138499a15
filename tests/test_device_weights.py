"""The lazy weight provider of the full-size parity tests hands the oracle exactly the tensors the packed model holds."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

import etx_megakernel_b200  # noqa: E402,F401
from etx_megakernel_b200.models import qwen as Q  # noqa: E402
from oracle import ref_decode as O  # noqa: E402
from tests.device_weights import DeviceWeights  # noqa: E402
from tests.golden.cases import SMALL_DENSE, SMALL_MOE  # noqa: E402


@pytest.mark.parametrize("od", [SMALL_MOE, SMALL_DENSE])
def test_lazy_provider_returns_the_packed_tensors(od):
    d = Q.Dims(**{f: getattr(od, f) for f in ("name", "H", "NH", "NKV", "HD", "INTER", "L", "V", "eps", "theta", "tie", "bias",
                                              "qk_norm", "moe", "E", "TOPK", "MI", "norm_topk")})
    W = O.SyntheticWeights(od, seed=4, gamma="normal")
    packed = {k: torch.from_numpy(np.ascontiguousarray(v).view(np.int16)).view(torch.bfloat16) for k, v in Q.pack_hf(d, W.get, 32).items()}
    for cache_bytes in (1 << 30, 0):                                        # everything cached / everything staged
        lazy = DeviceWeights(d, packed, cache_bytes=cache_bytes)
        for name, want in W.t.items():
            assert (name in lazy) or name == "lm_head.weight"
            got = lazy.get(name)
            if name == "model.embed_tokens.weight":
                assert np.array_equal(got[3], want[3])
            else:
                assert np.array_equal(np.asarray(got), want), name
        assert ("lm_head.weight" in lazy) == (not d.tie)
    # the oracle runs on it and gives the same token as on the original weights
    a = O.Ref(od, W, 16).step(5, 0)
    b = O.Ref(od, DeviceWeights(d, packed), 16).step(5, 0)
    assert a == b
