"""Weight pack files and golden token files in the reference's formats, so a directory prepared for the reference runs here.

`vl.bin` + `vl.manifest` (written by examples/vllm_llm/prep.py:71-150):
  * vl.bin: the packed bf16 tensors back to back, each starting on a 256-byte boundary;
  * vl.manifest: text lines `cfg <key> <int>`, `cfgf eps <float repr>`, `t <name> <byte offset> <element count>`;
    tensor names: embed, final_norm, lm_head (untied), cos_sin, and per layer `L<i>.ln1 ln2 wqkv [bqkv] [qn kn] wo`
    + `wr w13 w2` (MoE) or `wgu wd` (dense).  The packed shapes are those of `models.qwen.weight_shapes`.
Golden token files (`golden_c<context>.txt`, etx/models/llm/prep.py:237-238): three lines `prompt: <ids>`, `gen: <ids>`,
`margin: <floats>` -- the greedy continuation of a reference implementation with the top-1/top-2 logit margin of every
generated token; `check_golden` is the gate the reference applies (every token equal, except where the margin says the
reference itself was within rounding of a tie).

Nothing here needs a GPU; `read_vl` memory-maps the file, `to_device` uploads it.
"""
from __future__ import annotations

import re
from pathlib import Path

import numpy as np

from . import qwen as Q

ALIGN = 256
_CFG_KEYS = ("H", "NH", "NKV", "HD", "INTER", "L", "V", "tie", "bias", "qk_norm", "maxlen", "bytes", "moe", "E", "TOPK", "MI", "norm_topk")


def _file_name(name: str) -> str:
    """This package names layer tensors "<i>.<what>", the pack file "L<i>.<what>"."""
    m = re.fullmatch(r"(\d+)\.(\w+)", name)
    return f"L{m.group(1)}.{m.group(2)}" if m else name


def _our_name(name: str) -> str:
    m = re.fullmatch(r"L(\d+)\.(\w+)", name)
    return f"{m.group(1)}.{m.group(2)}" if m else name


def tensor_order(d: Q.Dims) -> list:
    """Names in the order the reference's packer writes them."""
    names = ["embed", "final_norm"] + ([] if d.tie else ["lm_head"]) + ["cos_sin"]
    for L in range(d.L):
        names += [f"{L}.ln1", f"{L}.ln2", f"{L}.wqkv"] + ([f"{L}.bqkv"] if d.bias else []) + ([f"{L}.qn", f"{L}.kn"] if d.qk_norm else [])
        names += [f"{L}.wo"] + ([f"{L}.wr", f"{L}.w13", f"{L}.w2"] if d.moe else [f"{L}.wgu", f"{L}.wd"])
    return names


def write_vl(out_dir, d: Q.Dims, packed: dict, maxlen: int) -> int:
    """packed: name -> uint16 array (bf16 bit patterns) with the shapes of weight_shapes(d, maxlen).  Returns the file size."""
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    want = Q.weight_shapes(d, maxlen)
    lines, off = [], 0
    with open(out / "vl.bin", "wb") as f:
        for name in tensor_order(d):
            a = np.ascontiguousarray(packed[name])
            if a.dtype != np.uint16 or tuple(a.shape) != tuple(want[name]):
                raise ValueError(f"{name}: expected uint16 {tuple(want[name])}, got {a.dtype} {a.shape}")
            pad = (-off) % ALIGN
            f.write(b"\0" * pad)
            off += pad
            f.write(a.tobytes())
            lines.append(f"t {_file_name(name)} {off} {a.size}")
            off += a.nbytes
    cfg = {"H": d.H, "NH": d.NH, "NKV": d.NKV, "HD": d.HD, "INTER": d.INTER, "L": d.L, "V": d.V, "tie": int(d.tie), "bias": int(d.bias),
           "qk_norm": int(d.qk_norm), "maxlen": maxlen, "bytes": off, "moe": int(d.moe), "E": d.E, "TOPK": d.TOPK, "MI": d.MI,
           "norm_topk": int(d.norm_topk)}
    text = "".join(f"cfg {k} {v}\n" for k, v in cfg.items()) + f"cfgf eps {float(d.eps)!r}\n" + "\n".join(lines) + "\n"
    (out / "vl.manifest").write_text(text)
    return off


def read_manifest(path) -> tuple:
    """(cfg: dict of ints plus float eps, tensors: file name -> (offset, elements))."""
    cfg, tensors = {}, {}
    for ln, line in enumerate(Path(path).read_text().splitlines(), 1):
        p = line.split()
        if not p:
            continue
        if p[0] == "cfg" and len(p) == 3:
            cfg[p[1]] = int(p[2])
        elif p[0] == "cfgf" and len(p) == 3:
            cfg[p[1]] = float(p[2])
        elif p[0] == "t" and len(p) == 4:
            tensors[p[1]] = (int(p[2]), int(p[3]))
        else:
            raise ValueError(f"{path}:{ln}: not a manifest line: {line!r}")
    return cfg, tensors


def read_vl(src_dir, theta: float = 1e6) -> tuple:
    """(Dims, maxlen, name -> uint16 array view of vl.bin) of a directory the reference's packer (or write_vl) made.

    The manifest carries no rope base (it is baked into the cos_sin table): `theta` only labels the Dims.  Model kinds
    this build has no tiles for are refused by name rather than run wrong."""
    src = Path(src_dir)
    cfg, tens = read_manifest(src / "vl.manifest")
    missing = [k for k in _CFG_KEYS if k not in cfg] + ([] if "eps" in cfg else ["eps"])
    if missing:
        raise ValueError(f"{src}/vl.manifest: missing cfg keys {missing}")
    for k in ("ln_norm", "sparsemixer", "bias_o", "bias_lm"):
        if cfg.get(k, 0):
            raise ValueError(f"{src}/vl.manifest: cfg {k} = 1 (LayerNorm / SparseMixer / output biases) is not supported by this build")
    d = Q.Dims(name=src.name, H=cfg["H"], NH=cfg["NH"], NKV=cfg["NKV"], HD=cfg["HD"], INTER=cfg["INTER"], L=cfg["L"], V=cfg["V"],
               eps=cfg["eps"], theta=theta, tie=bool(cfg["tie"]), bias=bool(cfg["bias"]), qk_norm=bool(cfg["qk_norm"]), moe=bool(cfg["moe"]),
               E=cfg["E"], TOPK=cfg["TOPK"], MI=cfg["MI"], norm_topk=bool(cfg["norm_topk"]))
    maxlen = cfg["maxlen"]
    size = (src / "vl.bin").stat().st_size
    if size != cfg["bytes"]:
        raise ValueError(f"{src}/vl.bin is {size} bytes, the manifest says {cfg['bytes']}")
    raw = np.memmap(src / "vl.bin", dtype=np.uint16, mode="r")
    out = {}
    for name, shape in Q.weight_shapes(d, maxlen).items():
        fn = _file_name(name)
        if fn not in tens:
            raise ValueError(f"{src}/vl.manifest: tensor {fn} is missing")
        off, n = tens[fn]
        if off % ALIGN or n != int(np.prod(shape)) or off + 2 * n > size:
            raise ValueError(f"{src}/vl.manifest: tensor {fn}: offset {off} / {n} elements do not fit shape {tuple(shape)} (256-byte aligned, inside the file)")
        out[name] = raw[off // 2: off // 2 + n].reshape(shape)
    extra = sorted(set(map(_our_name, tens)) - set(out))
    if extra:
        raise ValueError(f"{src}/vl.manifest: tensors this build has no use for: {extra[:6]} (a model kind it does not support)")
    return d, maxlen, out


def to_device(packed: dict, device):
    """uint16 views -> bf16 device tensors (one host copy per tensor)."""
    import torch
    return {k: torch.from_numpy(np.array(v, dtype=np.uint16).view(np.int16)).to(device).view(torch.bfloat16) for k, v in packed.items()}


# ---------------------------------------------------------------------------------------------- golden token files
def write_golden(path, prompt, gen, margins) -> None:
    Path(path).write_text("prompt: " + " ".join(str(int(t)) for t in prompt) + "\n" + "gen: " + " ".join(str(int(t)) for t in gen) + "\n"
                          + "margin: " + " ".join(f"{float(m):.4f}" for m in margins) + "\n")


def read_golden(path) -> tuple:
    """(prompt ids, generated ids, margins)."""
    rows = {}
    for line in Path(path).read_text().splitlines():
        if ":" in line:
            k, v = line.split(":", 1)
            rows[k.strip()] = v.split()
    if "prompt" not in rows or "gen" not in rows:
        raise ValueError(f"{path}: needs a 'prompt:' and a 'gen:' line")
    gen = [int(t) for t in rows["gen"]]
    margins = [float(t) for t in rows.get("margin", [])] or [float("inf")] * len(gen)
    if len(margins) != len(gen):
        raise ValueError(f"{path}: {len(gen)} generated tokens but {len(margins)} margins")
    return [int(t) for t in rows["prompt"]], gen, margins


def check_golden(generated, gen, margins, tie_margin: float = 0.0) -> list:
    """Differences between `generated` and the golden continuation that the golden's own margins do not excuse.

    A greedy run is compared token by token up to the first difference (after it the contexts differ); that difference
    is excused when the reference's top-1/top-2 margin there is <= tie_margin.  Returns a list of messages (empty: pass)."""
    out = []
    if len(generated) < len(gen):
        out.append(f"only {len(generated)} of {len(gen)} tokens generated")
    for i, (a, b) in enumerate(zip(generated, gen)):
        if int(a) != int(b):
            if margins[i] > tie_margin:
                out.append(f"token {i}: generated {int(a)}, golden {int(b)} (golden margin {margins[i]:.4f} > {tie_margin})")
            break
    return out
