"""Built-in tiles of the B200 megakernel as ETX ops (argument-block layouts + export tables)."""
from . import attn, attnprep, batch, gemv, mla, topk


def all_entries() -> dict:
    out = {}
    for m in (gemv, topk, attnprep, attn, batch, mla):
        out.update(m.import_entries())
    return out
