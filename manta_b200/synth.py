"""Seeded synthetic candidate sets, generated on the device in row chunks.

Rows are N(0,1) entries (optionally L2-normalised), rounded to f16, then packed by the library's own
quantiser kernels.  Chunk c (rows [c*CHUNK, (c+1)*CHUNK)) is drawn from a generator seeded with
``seed + c``, so any shard can produce exactly its own rows and a sharded set equals the unsharded one.
These stand in for the BEIR-format corpora the reference evaluates on, which are not available offline.
"""
from __future__ import annotations

import torch

CHUNK = 1 << 18  # rows per generator seed
SEED_DOCS = 0x4D414E54
SEED_QUERIES = SEED_DOCS + 1
SEED_TOKENS = SEED_DOCS + 2
SEED_WEIGHTS = SEED_DOCS + 3


def _chunk_f16(seed: int, chunk: int, cols: int, normalise: bool, device) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(seed + chunk)
    x = torch.randn((CHUNK, cols), generator=g, device=device, dtype=torch.float32)
    if normalise:
        x = x / x.norm(dim=1, keepdim=True).clamp_min(1e-30)
    return x.to(torch.float16)


def rows_f16(row_begin: int, row_end: int, cols: int, normalise: bool = True, seed: int = SEED_DOCS,
             device="cuda") -> torch.Tensor:
    """f16 rows [row_begin, row_end) of the seeded set."""
    out = torch.empty((row_end - row_begin, cols), dtype=torch.float16, device=device)
    c0, c1 = row_begin // CHUNK, (row_end + CHUNK - 1) // CHUNK
    for c in range(c0, c1):
        x = _chunk_f16(seed, c, cols, normalise, device)
        lo, hi = max(row_begin, c * CHUNK), min(row_end, (c + 1) * CHUNK)
        out[lo - row_begin:hi - row_begin] = x[lo - c * CHUNK:hi - c * CHUNK]
    return out


def queries_f16(nq: int, cols: int, normalise: bool = True, seed: int = SEED_QUERIES, device="cuda") -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    x = torch.randn((nq, cols), generator=g, device=device, dtype=torch.float32)
    if normalise:
        x = x / x.norm(dim=1, keepdim=True).clamp_min(1e-30)
    return x.to(torch.float16)


def packed_candidates(rt, layout: str, row_begin: int, row_end: int, cols: int, normalise: bool = True,
                      seed: int = SEED_DOCS, device="cuda"):
    """Generates rows [row_begin, row_end) chunk by chunk and packs them on the device.
    Returns (data, scales) device tensors in the layout's packed form (scales None for f16)."""
    rows = row_end - row_begin
    stream = torch.cuda.ExternalStream(rt.stream)
    with torch.cuda.stream(stream):
        if layout == "f16":
            data = torch.empty((rows, cols), dtype=torch.float16, device=device)
            scales = None
        elif layout == "q8":
            data = torch.empty((rows, cols), dtype=torch.int8, device=device)
            scales = torch.empty(rows, dtype=torch.float32, device=device)
        else:
            data = torch.empty((rows, cols // 2), dtype=torch.uint8, device=device)
            scales = torch.empty((rows, cols // 32), dtype=torch.int16, device=device)
        c0, c1 = row_begin // CHUNK, (row_end + CHUNK - 1) // CHUNK
        for c in range(c0, c1):
            x = _chunk_f16(seed, c, cols, normalise, device)
            lo, hi = max(row_begin, c * CHUNK), min(row_end, (c + 1) * CHUNK)
            src = x[lo - c * CHUNK:hi - c * CHUNK].contiguous()
            n = hi - lo
            o = lo - row_begin
            if layout == "f16":
                data[o:o + n] = src
            elif layout == "q8":
                rt.pack_q8_rows_device(src, True, n, cols, data[o:o + n], scales[o:o + n])
            else:
                rt.pack_q4_b32_device(src, True, n, cols, data[o:o + n], scales[o:o + n])
            stream.synchronize()  # src is released after the pack kernel has consumed it
    return data, scales


def embed_weights_f16(vocab: int, dim: int, out_dim: int, seed: int = SEED_WEIGHTS, device="cuda"):
    """token_embedding f16[vocab, dim] ~ N(0, 0.02) and projection f16[dim, out_dim] ~ N(0, 0.05)."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    table = (torch.randn((vocab, dim), generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.float16)
    proj = (torch.randn((dim, out_dim), generator=g, device=device, dtype=torch.float32) * 0.05).to(torch.float16)
    return table, proj


def token_batches(nsets: int, batch: int, seq: int, vocab: int, min_len: int = 16, seed: int = SEED_TOKENS, device="cuda"):
    """tokens i32[nsets, batch, seq] uniform in [0, vocab) and the mask of lengths uniform in min_len..seq."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    tokens = torch.randint(0, vocab, (nsets, batch, seq), generator=g, device=device, dtype=torch.int32)
    lengths = torch.randint(min(min_len, seq), seq + 1, (nsets, batch, 1), generator=g, device=device, dtype=torch.int32)
    mask = (torch.arange(seq, device=device, dtype=torch.int32).view(1, 1, seq) < lengths).to(torch.int32)
    return tokens, mask
