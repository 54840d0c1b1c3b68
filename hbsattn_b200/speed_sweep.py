"""Runtime comparison on the reference's own benchmark shapes, written in the reference's result format.

    python -m hbsattn_b200.speed_sweep --causal --unit_seqlen 8192 --sparse_ratio 0.9 [--nruns 15 --nwarmup 5]
        [--headdim 128 --nheads 32 --batch_size 8 --save_benchmark_to_file results.json --reference_dir DIR]

Same flags, same workload (fixed 128x128 blocks, batch of equal-length samples, Bernoulli block mask with the first
in-sample k-block forced True) and same JSON layout as the reference's speed script (test/test_speedup.py:38-50,
:88-115, :208-238): a list of entries with the keys ``flash_attn_base_result``, ``hbsattn(our fix)``,
``hbsattn(our auto)``, ``hanlab_block-sparse-attn``, ``flexattention`` plus ``unit_seqlen``, ``headdim``, ``nhead_q``,
``causal``, ``sparse_ratio``; every result is ``{runtime_mean, runtime_std, runtime_min, runtime_max, all_times,
error}`` (hbsattn/benchmark.py:98-105), so the reference's plot script (test/plot_benchmark_runtime.py:31-80) reads the
file unchanged.  A configuration that is already in the file is skipped (test/test_speedup.py:53-69).

What fills the columns: the two ``hbsattn`` columns are THIS package's operator with ``tile_mode`` ``'fix'`` / ``'auto'``;
``flash_attn_base_result`` is dense FlashAttention (``flash_attn_varlen_func``) and ``flexattention`` is
``torch.nn.attention.flex_attention`` with a block mask, each when importable and runnable on this GPU (else ``{}``, as
the reference does on an exception); the Han-lab library is not installed anywhere this runs, its column stays ``{}``.
With ``--reference_dir`` (the directory of an installed reference package, e.g. baseline/_ref) two more keys,
``reference triton(fix)`` and ``reference triton(auto)``, hold the unmodified reference operator.
Timing is the reference's: host wall clock around the call with a device synchronise on both sides.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np
import torch


def timed(fn, n_runs, n_warmup):
    """hbsattn/benchmark.py:50-105 without the printing: n_runs calls, the first n_warmup discarded."""
    times = []
    for i in range(n_runs):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        fn()
        torch.cuda.synchronize()
        if i >= n_warmup:
            times.append(time.perf_counter() - t0)
    t = np.array(times)
    return {"runtime_mean": float(t.mean()), "runtime_std": float(t.std()), "runtime_min": float(t.min()),
            "runtime_max": float(t.max()), "all_times": t.tolist(), "error": None}


def guarded(name, fn, n_runs, n_warmup):
    try:
        return timed(fn, n_runs, n_warmup)
    except Exception as e:                          # the reference prints and records {} (test/test_speedup.py:141-143)
        print(f"Error benchmarking {name}: {type(e).__name__}: {e}"[:300])
        return {}


def already_there(path, cfg):
    if not path or not os.path.exists(path):
        return False
    with open(path) as f:
        for entry in json.load(f):
            if all(entry.get(key) == val for key, val in cfg.items()):
                return True
    return False


def append_result(path, entry):
    data = []
    if os.path.exists(path):
        with open(path) as f:
            data = json.load(f)
    data.append(entry)
    with open(path, "w") as f:
        json.dump(data, f, indent=4)
    return len(data)


def build_inputs(args, device):
    """test/test_speedup.py:88-115: equal-length samples, 128x128 blocks, Bernoulli(1 - sparse_ratio) mask with the first
    k-block of every q-block's own sample forced True."""
    from .utils import calculate_blocks
    bs, L, H, d = args.batch_size, args.unit_seqlen, args.nheads, args.headdim
    cu = torch.arange(0, bs + 1, dtype=torch.int32, device=device) * L
    q = torch.randn(bs * L, H, d, device=device, dtype=torch.bfloat16)
    k = torch.randn(bs * L, H, d, device=device, dtype=torch.bfloat16)
    v = torch.randn(bs * L, H, d, device=device, dtype=torch.bfloat16)
    mq = calculate_blocks(cu, 128)
    mk = calculate_blocks(cu, 128)
    mask = torch.rand(H, mq[0], mk[0], device=device) < 1 - args.sparse_ratio
    per = (L + 127) // 128
    qi = torch.arange(mq[0], device=device)
    mask[:, qi, (qi // per) * per] = True
    return q, k, v, cu, mask, mq, mk


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--causal", action="store_true", default=False)
    ap.add_argument("--softmax_scale", type=float, default=None)
    ap.add_argument("--nruns", type=int, default=2)
    ap.add_argument("--nwarmup", type=int, default=1)
    ap.add_argument("--headdim", type=int, default=128)
    ap.add_argument("--unit_seqlen", type=int, default=256)
    ap.add_argument("--nheads", type=int, default=32)
    ap.add_argument("--batch_size", type=int, default=8)
    ap.add_argument("--save_benchmark_to_file", type=str, default="./benchmark_all_results.json")
    ap.add_argument("--sparse_ratio", type=float, default=0.3)
    ap.add_argument("--reference_dir", type=str, default=None, help="directory that holds an installed reference package (optional)")
    ap.add_argument("--no_flex", action="store_true", help="skip FlexAttention (its compile step takes minutes at long sequences)")
    args = ap.parse_args(argv)
    cfg = {"unit_seqlen": args.unit_seqlen, "headdim": args.headdim, "nhead_q": args.nheads, "causal": args.causal,
           "sparse_ratio": args.sparse_ratio}
    if already_there(args.save_benchmark_to_file, cfg):
        print(f"[INFO] Configuration already exists in {args.save_benchmark_to_file}: {cfg}\n[INFO] Skipping benchmark...")
        return 0
    if not torch.cuda.is_available():
        raise RuntimeError("the sweep needs a CUDA device: hbsattn_b200 has no CPU path")
    from . import HBSAttention
    dev = torch.device("cuda", torch.cuda.current_device())
    q, k, v, cu, mask, mq, mk = build_inputs(args, dev)
    L, scale = args.unit_seqlen, args.softmax_scale
    entry = dict(cfg)

    def ours(mode):
        return lambda: HBSAttention(q, k, v, cu, cu, mask, 128, 128, args.causal, scale, mode, *mq, *mk)
    entry["hbsattn(our fix)"] = guarded("hbsattn_b200 fix", ours("fix"), args.nruns, args.nwarmup)
    entry["hbsattn(our auto)"] = guarded("hbsattn_b200 auto", ours("auto"), args.nruns, args.nwarmup)

    def flash():
        from flash_attn import flash_attn_varlen_func
        return flash_attn_varlen_func(q, k, v, cu, cu, L, L, 0.0, scale, args.causal)
    entry["flash_attn_base_result"] = guarded("FlashAttention", flash, args.nruns, args.nwarmup)
    entry["hanlab_block-sparse-attn"] = {}

    if args.no_flex:
        entry["flexattention"] = {}
    else:
        def make_flex():
            from torch.nn.attention.flex_attention import create_block_mask, flex_attention
            bs, H, d = args.batch_size, args.nheads, args.headdim
            per = (L + 127) // 128
            planes = torch.stack([mask[:, b * per:(b + 1) * per, b * per:(b + 1) * per] for b in range(bs)])   # [B, H, per, per]

            def mask_mod(b, h, qi, ki):
                keep = planes[b, h, qi // 128, ki // 128]
                return keep & (qi >= ki) if args.causal else keep
            bm = create_block_mask(mask_mod, bs, H, L, L, device=dev, BLOCK_SIZE=128)
            qp, kp, vp = (t.view(bs, L, H, d).permute(0, 2, 1, 3) for t in (q, k, v))
            fa = torch.compile(flex_attention)
            return lambda: fa(qp, kp, vp, block_mask=bm, scale=scale)
        try:
            entry["flexattention"] = guarded("FlexAttention", make_flex(), args.nruns, args.nwarmup)
        except Exception as e:
            print(f"Error benchmarking flexattention: {type(e).__name__}: {e}"[:300])
            entry["flexattention"] = {}

    if args.reference_dir:
        try:
            sys.path.insert(0, args.reference_dir)
            import hbsattn as ref                                  # the unmodified reference package
            sys.path.remove(args.reference_dir)
            for mode in ("fix", "auto"):
                entry[f"reference triton({mode})"] = guarded(
                    f"reference {mode}", lambda mode=mode: ref.HBSAttention(q, k, v, cu, cu, mask, 128, 128, args.causal, scale, mode, *mq, *mk),
                    args.nruns, args.nwarmup)
        except Exception as e:
            print(f"Error loading the reference: {type(e).__name__}: {e}"[:300])

    if args.save_benchmark_to_file:
        n = append_result(args.save_benchmark_to_file, entry)
        print(f"\n Benchmark results saved to {args.save_benchmark_to_file}\n   Total entries in file: {n}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
