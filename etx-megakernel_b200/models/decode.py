"""DecodeProgram: a Qwen-family decode session on one GPU -- weights, buffers, plan, session, token loop.

The host lifecycle of the reference's run binary (examples/vllm_llm/host.hip:126-1159): upload packed weights,
allocate per-request activations and paged KV caches, fill one argument block per grid instance, set up the session,
then one launch per token with the next token written on the device by the argmax tile.
"""
from __future__ import annotations

import numpy as np
import torch

from ..machine import load_machine
from ..passes import PassOptions, compile_graph
from ..runtime import ExchangeRegion, Session
from . import qwen as Q

_DT = {"bf16": torch.bfloat16, "f32": torch.float32, "i32": torch.int32, "i64": torch.int64}


def random_packed_weights(d: Q.Dims, maxlen: int, device, seed: int = 0, std: float = 0.02, gamma: str = "ones") -> dict:
    """Seeded random-init weights generated on the device, already in the packed layouts: linear / embedding weights
    ~ N(0, std) rounded to bf16, norm gammas 1.0 ("ones") or ~ N(0, std) ("normal")."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    out = {}
    for name, shape in Q.weight_shapes(d, maxlen).items():
        if name == "cos_sin":
            out[name] = torch.from_numpy(Q.rope_table(d.theta, d.HD, maxlen).view(np.int16)).to(device).view(torch.bfloat16)
            continue
        is_gamma = name.rsplit(".", 1)[-1] in ("ln1", "ln2", "qn", "kn", "final_norm")
        t = torch.empty(shape, dtype=torch.bfloat16, device=device)
        if is_gamma and gamma == "ones":
            t.fill_(1.0)
        else:
            t.normal_(0.0, std, generator=gen)
        out[name] = t
    return out


def to_device_weights(packed: dict, device) -> dict:
    """uint16 numpy arrays (Q.pack_hf) -> bf16 device tensors."""
    return {k: torch.from_numpy(np.ascontiguousarray(v).view(np.int16)).to(device).view(torch.bfloat16) for k, v in packed.items()}


class DecodeProgram:
    def __init__(self, dims: Q.Dims, weights: dict, device: int = 0, maxlen: int = 1072, steps: int | None = None, machine="b200",
                 fold_topk: bool = True, fused_attn: bool | str = True, workers: int | None = None, ranks: int = 1, rank: int = 0,
                 flagged: bool = False):
        """ranks > 1: rank `rank` of a model sharded `ranks` ways -- `dims` and `weights` are the rank's shard
        (Q.shard_dims / Q.shard_weights); call connect() with every rank's `region.handle` before the first step."""
        self.d, self.maxlen = dims, maxlen
        self.ranks, self.rank, self.region, self.xaddr = ranks, rank, None, {}
        self.dev = torch.device("cuda", device)
        self.machine = load_machine(machine) if isinstance(machine, str) else machine
        self.steps = steps or maxlen
        self.w = weights
        want = Q.weight_shapes(dims, maxlen)
        for k, shp in want.items():
            if k not in weights or tuple(weights[k].shape) != tuple(shp):
                raise ValueError(f"weight {k}: expected shape {shp}, got {tuple(weights[k].shape) if k in weights else None}")
        sz = Q.size_for(dims, self.machine, maxlen)
        self.buf = {n: torch.zeros(shape, dtype=_DT[dt], device=self.dev) for n, (shape, dt) in Q.buffer_shapes(dims, maxlen, self.steps, sz.parts).items()}
        self.buf["block_tables"].copy_(torch.arange(self.buf["block_tables"].numel(), dtype=torch.int32))
        self.vl = torch.zeros(1, dtype=torch.int64, device=self.dev)

        if ranks > 1 or flagged:
            self.region = ExchangeRegion(Q.exchange_bytes(dims, ranks), device)      # the blocks of flagged rows the ranks publish into
            self.xaddr = {"xrows": self.region.ptr}

        def ptr(name):
            if name in self.xaddr:
                return self.xaddr[name]
            t = self.buf.get(name)
            if t is None:
                t = self.w[name]
            return t.data_ptr()
        self.graph, self.pool, self.sizing = Q.build_graph(dims, ptr, maxlen, self.machine, fold_topk=fold_topk, fused_attn=fused_attn,
                                                              ranks=ranks, rank=rank, flagged=flagged)
        pool = self.pool.bytes()
        self.plan = compile_graph(self.graph, self.machine, {"POOL": len(pool)}, options=PassOptions(workers=workers))
        self.session = Session(self.plan, {"vl": self.vl}, pool, device)
        b = self.buf
        self.session.set_step(tok=0, pos=0, write_next=0, H=dims.H, V=dims.lm_rows, nrep=1, embed=self.w["embed"], resid=b["resid"],
                              positions=b["positions"], seq_lens=b["seq_lens"], slot_mapping=b["slot_mapping"], logits=b["logits"],
                              token_in=b["token_in"], token_out=b["token_out"], token_time=b["token_time"])
        if flagged and ranks == 1:
            self.session.set_exchange(0, 1, self.region)            # one rank: nothing to connect, the region is its own

    def connect(self, handles: list):
        """handles[r] = rank r's `region.handle` (all-gathered by the caller).  After this, and a barrier so that no
        rank steps before every rank is connected, the ranks step in lock step."""
        self.region.connect(self.rank, handles)
        self.session.set_exchange(self.rank, self.ranks, self.region)
        if self.d.VL:                                            # lm_head split by vocabulary: the argmax tile exchanges (max, index) pairs
            self.session.set_option("exchange_argmax_offset", Q.argmax_offset(self.d, self.ranks))

    # ---- KV cache helpers (contiguous [ctx][NKV][HD] <-> the paged layout)
    def load_kv(self, layer: int, K: np.ndarray, V: np.ndarray):
        """Pre-fill positions 0..ctx-1 of one layer from contiguous float32 (bf16-exact) arrays."""
        ctx, nkv, hd = K.shape
        kc, vc = self.buf["kc"][layer], self.buf["vc"][layer]
        Kt = torch.from_numpy(np.ascontiguousarray(K)).to(self.dev).to(torch.bfloat16)
        Vt = torch.from_numpy(np.ascontiguousarray(V)).to(self.dev).to(torch.bfloat16)
        pad = (-ctx) % Q.BS
        if pad:
            Kt = torch.cat([Kt, torch.zeros(pad, nkv, hd, dtype=Kt.dtype, device=self.dev)])
            Vt = torch.cat([Vt, torch.zeros(pad, nkv, hd, dtype=Vt.dtype, device=self.dev)])
        nb = Kt.shape[0] // Q.BS
        kc[:nb] = Kt.view(nb, Q.BS, nkv, hd // Q.X, Q.X).permute(0, 2, 3, 1, 4)
        vc[:nb] = Vt.view(nb, Q.BS, nkv, hd).permute(0, 2, 3, 1)

    def read_kv(self, layer: int, ctx: int):
        kc, vc = self.buf["kc"][layer].float().cpu().numpy(), self.buf["vc"][layer].float().cpu().numpy()
        nb, nkv, hdx, bs, x = kc.shape
        K = kc.transpose(0, 3, 1, 2, 4).reshape(nb * bs, nkv, hdx * x)[:ctx]
        V = vc.transpose(0, 3, 1, 2).reshape(nb * bs, nkv, hdx * x)[:ctx]
        return K, V

    def read(self, name: str) -> np.ndarray:
        t = self.buf[name]
        return (t.float() if t.dtype == torch.bfloat16 else t).cpu().numpy()

    # ---- stepping
    def step(self, t: int, pos: int, write_next: bool, wait: bool = True, unfused: bool = False):
        """One decode step; unfused=True runs it as one kernel launch per grid (the baseline the single launch is compared with)."""
        self.session.set_step(tok=t, pos=pos, write_next=int(write_next))
        if unfused:
            self.session.launch_unfused()
            if wait:
                self.session.wait(60.0)
        elif wait:
            self.session.run(60.0)
        else:
            self.session.launch()

    def generate(self, prompt, n_gen: int, start_pos: int = 0, sync_every: int = 64, unfused: bool = False):
        """Feed `prompt` token by token (positions start_pos ...), then n_gen greedy tokens; the next token never leaves
        the device.  Returns the n_gen generated ids (the argmax after the last prompt token is the first)."""
        prompt = [int(x) for x in prompt]
        n = len(prompt) + n_gen - 1
        if n + 2 > self.buf["token_in"].numel() or start_pos + n > self.maxlen:
            raise ValueError("sequence longer than the session was sized for")
        tin = torch.zeros_like(self.buf["token_in"])
        tin[:len(prompt)] = torch.tensor(prompt, dtype=torch.int32)
        self.buf["token_in"].copy_(tin)
        torch.cuda.synchronize(self.dev)
        for t in range(n):
            self.step(t, start_pos + t, write_next=t + 1 >= len(prompt), wait=(t % sync_every == sync_every - 1) or t == n - 1, unfused=unfused)
        return self.buf["token_out"][len(prompt) - 1:n].cpu().numpy()

    def generate_host(self, prompt, n_gen: int, start_pos: int = 0):
        """The same through host buffers: every step's token goes host -> device and its result device -> host."""
        toks, ms = self.session.decode_host(np.asarray(prompt, np.int32), len(prompt) + n_gen - 1, start_pos)
        return toks[len(prompt) - 1:], ms

    def close(self):
        """Sharded: every rank must have finished its last step (synchronise, then a barrier) before any rank closes --
        a running peer still stores into this rank's region."""
        self.session.close()
        if self.region is not None:
            self.region.close()
            self.region = None
