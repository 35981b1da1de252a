"""Kernel-only driver of the sequence attention kernels (also used under ncu):

    python profiles/run_seq_attention.py [chunk|decode] [tokens] [heads] [kv_heads] [head_dim]

chunk: one prompt of `tokens` positions through attn_chunk_kernel (global, zero sink), bf16 cache rows.
decode: one token at context `tokens` through attn_decode_kernel.  Prints CUDA-event times after warm-up."""
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from cold_compress_b200 import seq_ops  # noqa: E402
from cold_compress_b200.cache import get_cache_constructor  # noqa: E402

mode = sys.argv[1] if len(sys.argv) > 1 else "chunk"
P, H, G, D = (int(v) for v in (sys.argv[2:6] + ["4096", "16", "4", "128"][len(sys.argv) - 2:]))
dev = torch.device("cuda", 0)
gen = torch.Generator(device=dev).manual_seed(0)
q = torch.randn(P, H, D, device=dev, generator=gen)
k = torch.randn(P, G, D, device=dev, generator=gen).to(torch.bfloat16)
v = torch.randn(P, G, D, device=dev, generator=gen).to(torch.bfloat16)
y = torch.empty(P, H, D, device=dev, dtype=torch.bfloat16)
ctor, _ = get_cache_constructor("full")
with torch.device(dev):
    cache = ctor(1, G, D, torch.bfloat16, max_cache_length=P + 8, global_tokens=0, max_seq_length=P + 8, cache_bits=None)
ip0 = torch.zeros(1, dtype=torch.int32, device=dev)
args = (q, k, v, cache.k_cache, cache.v_cache, cache.pos, cache.mask, cache.cache_cts, ip0, y, None, 0, 2, D ** -0.5)


def timed(fn, warm, n):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(n):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / n


if mode == "chunk":
    ms = timed(lambda: seq_ops.seq_attention(*args, seq_ops.ATTN_CHUNK, None), 1, 2)
    flop = 4 * (P * (P + 1) / 2) * D * H
    print(f"attn_chunk_kernel P={P} H={H} G={G} D={D}: {ms:.3f} ms, {flop / ms / 1e9:.2f} TFLOP/s fp32 (causal work only)")
else:
    if P <= 8192:
        seq_ops.seq_attention(*args, seq_ops.ATTN_CHUNK, None)
    seq_ops.seq_attention(*args, seq_ops.ATTN_APPEND_ONLY, None)
    ipd = torch.tensor([P], dtype=torch.int32, device=dev)
    ws = cache._sequence_workspace(H, 0)
    dargs = (q[:1], k[:1], v[:1], cache.k_cache, cache.v_cache, cache.pos, cache.mask, cache.cache_cts, ipd, y[:1], None, 0, 2, D ** -0.5)
    graph = torch.cuda.CUDAGraph()
    seq_ops.seq_attention(*dargs, seq_ops.ATTN_DECODE, ws)
    torch.cuda.synchronize()
    with torch.cuda.graph(graph):
        for _ in range(20):
            seq_ops.seq_attention(*dargs, seq_ops.ATTN_DECODE, ws)
    ms = timed(graph.replay, 2, 5) / 20
    nbytes = 2 * G * P * D * 2
    print(f"attn_decode_kernel ctx={P} H={H} G={G} D={D}: {ms * 1e3:.2f} us per launch (graph of 20), "
          f"{nbytes / ms / 1e6:.1f} GB/s of live K/V rows")
