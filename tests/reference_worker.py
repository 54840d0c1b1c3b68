"""Runs the UNMODIFIED reference operator (its Triton kernels, from baseline/_ref) on inputs stored in a file and
stores its outputs (run as a script by tests/test_gpu_vs_reference.py, in a process of its own so that nothing the
reference does can disturb the test process).

    python tests/reference_worker.py <in.pt> <out.pt>

in.pt: {"cases": [{"q","k","v","cu_q","cu_k","mask","qbs","kbs","causal","scale","modes"}...]} with CPU tensors."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch


def main():
    import baseline
    ref = baseline.load_reference()
    from hbsattn.utils import calculate_blocks
    assert os.path.abspath(ref.__file__).startswith(baseline.REF_DIR)
    cases = torch.load(sys.argv[1])["cases"]
    dev = torch.device("cuda", 0)
    outs = []
    for c in cases:
        q, k, v, cu_q, cu_k, mask = (c[n].to(dev) for n in ("q", "k", "v", "cu_q", "cu_k", "mask"))
        mq = calculate_blocks(cu_q, c["qbs"])
        mk = calculate_blocks(cu_k, c["kbs"])
        res = {}
        for mode in c["modes"]:
            try:
                o = ref.HBSAttention(q, k, v, cu_q, cu_k, mask, c["qbs"], c["kbs"], c["causal"], c["scale"], mode, *mq, *mk)
                torch.cuda.synchronize()
                res[mode] = o.cpu()
            except Exception as e:                      # e.g. the compiler of this image cannot build the kernel for sm_100
                res[mode] = f"{type(e).__name__}: {e}"[:500]
        outs.append(res)
    torch.save({"outs": outs}, sys.argv[2])


if __name__ == "__main__":
    main()
