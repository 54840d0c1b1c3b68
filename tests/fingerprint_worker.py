"""Runs one benchmark workload through HBSAttention a number of times and stores a fingerprint of every output
(run as a script by tests/test_gpu_strict_order.py; which build of the library is loaded is decided by the
HBSATTN_B200_LIBRARY environment variable of the process).

    python tests/fingerprint_worker.py <workload> <repeats> <out.pt>

The fingerprint of an output [total_q, nhead_q, headdim] is one int64 per token: the 16-bit patterns of the token's
values weighted with fixed odd numbers and summed, so that two outputs have equal fingerprints only if they are
bit-identical (up to collisions of a 64-bit checksum)."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch


def fingerprint(out: torch.Tensor) -> torch.Tensor:
    flat = out.reshape(out.shape[0], -1)
    g = torch.Generator(device="cpu").manual_seed(1234)
    w = (torch.randint(1, 2 ** 31, (flat.shape[1],), generator=g, dtype=torch.int64) * 2 + 1).to(out.device)
    parts = []
    for r0 in range(0, flat.shape[0], 8192):
        bits = flat[r0:r0 + 8192].view(torch.int16).to(torch.int64)
        parts.append((bits * w).sum(dim=1))
    return torch.cat(parts).cpu()


def main():
    workload, repeats, out_path = sys.argv[1], int(sys.argv[2]), sys.argv[3]
    import bench
    import hbsattn_b200 as hb
    dev = torch.device("cuda", 0)
    wl = bench.make_workload(workload, 0, dev)
    w = wl["w"]
    hb.set_kernel_family("sm100")
    prints = []
    for _ in range(repeats):
        out = hb.HBSAttention(wl["q"], wl["k"], wl["v"], wl["cu_q_t"], wl["cu_k_t"], wl["mask"], w["qbs"], w["kbs"], w["causal"], None)
        assert hb.last_status()[0] == 0
        prints.append(fingerprint(out))
        del out
    from hbsattn_b200 import _lib
    torch.save({"prints": prints, "library": _lib.LIB_PATH}, out_path)


if __name__ == "__main__":
    main()
