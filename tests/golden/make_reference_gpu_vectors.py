"""Record outputs of the reference's own CUDA kernels, run on a GPU, as golden vectors.

Needs the reference built by oracle/build_reference.py (oracle/_ref/int4matmul_ref*.so) and a CUDA device:

    python tests/golden/make_reference_gpu_vectors.py OUTPUT.npz

For seeded problems (inputs are regenerated from the seed by oracle.reference_oracle.make_problem, so only
the outputs are stored) it runs the reference's `quant_matmul` (matvec and matmul routes, every supported
format) and `weight_matrix_packing`, and saves what they returned.  The stored file is copied to
tests/golden/reference_gpu_vectors.npz; tests then check the CPU oracle (no GPU needed) and the product's
kernels (GPU) against it.  Inputs are valid by construction (16 kept weights in every 32-block, fp16
activations, supported bit / sparsity combinations), so none of the reference's device asserts can fire.
"""
import glob
import importlib.util
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import reference_oracle as oracle  # noqa: E402

# (bits, sparse, N, S, M, group, seed)
CASES = [
    (4, False, 256, 128, 1, 64, 101), (4, False, 1024, 256, 1, 128, 102), (4, False, 256, 128, 70, 64, 103),
    (4, False, 512, 192, 5, 128, 104), (4, True, 256, 128, 1, 64, 105), (4, True, 512, 128, 70, 64, 106),
    (2, False, 256, 128, 1, 64, 107), (2, False, 256, 128, 70, 64, 108),
    (3, False, 256, 128, 70, 64, 109), (3, False, 512, 192, 130, 128, 110),
]
# the reference's dense int3 matvec kernel is only run when its build notes say it assembled with optimisation
INT3_MATVEC_CASE = (3, False, 256, 128, 1, 64, 111)
# exponent coding (negative scales select it, matmul.cuh:127-136, 414-428): whole aligned 32-column runs of a group
# switch together, as the reference's warp-uniform branch requires
EXPONENT_CASES = [(4, False, 256, 128, 1, 64, 121), (4, False, 256, 128, 70, 64, 122), (2, False, 256, 128, 70, 64, 123),
                  (4, True, 256, 128, 70, 64, 124)]


def load_reference():
    cand = glob.glob(os.path.join(ROOT, "oracle", "_ref", "int4matmul_ref*.so"))
    if not cand:
        raise SystemExit("oracle/_ref/int4matmul_ref*.so is missing: run oracle/build_reference.py where the reference is mounted")
    spec = importlib.util.spec_from_file_location("int4matmul_ref", cand[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(out_path):
    ref = load_reference()
    dev = "cuda:0"
    blob = {}
    cases = [c + (False,) for c in list(CASES) + [INT3_MATVEC_CASE]] + [c + (True,) for c in EXPONENT_CASES]
    for bits, sparse, n, s, m, g, seed, expo in cases:
        p = oracle.make_problem(bits, n, s, m, g, sparse=sparse, seed=seed, exponent_frac=0.5 if expo else 0.0)
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
        tag = f"b{bits}_{'sp' if sparse else 'dn'}_n{n}_s{s}_m{m}_g{g}_seed{seed}" + ("_exp" if expo else "")
        if sparse:
            # the packer: uint8 (S, N) weights and mask -> compacted words + bit mask
            wt = torch.empty((n // 16, s), dtype=torch.int32, device=dev)
            mk = torch.empty((n // 32, s), dtype=torch.int32, device=dev)
            ref.weight_matrix_packing(wt, mk, t(np.ascontiguousarray(p["q"].T)), t(np.ascontiguousarray(p["keep"].T).astype(np.uint8)))
            torch.cuda.synchronize()
            blob[tag + "_packed"] = wt.cpu().numpy()
            blob[tag + "_mask"] = mk.cpu().numpy()
        outs = torch.zeros((1, m, s), dtype=torch.float16, device=dev)
        ref.quant_matmul(bits, outs, t(p["matrix"]), t(p["x"]), t(p["scales"]), t(p["zeros"]), g,
                         t(p["mask"]) if sparse else None)
        torch.cuda.synchronize()
        blob[tag + "_out"] = outs.cpu().numpy()
        print(tag, "ok")
    np.savez_compressed(out_path, **blob)
    print("wrote", out_path)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_reference_gpu_vectors.py OUTPUT.npz")
    main(sys.argv[1])
