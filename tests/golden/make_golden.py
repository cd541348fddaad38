"""Generate the golden vectors under tests/golden/ from the reference's own Python helpers.

Run once in a container that has the reference checkout (it cannot travel with the repo):

    python tests/golden/make_golden.py /path/to/int4matmul_kernels

It imports the reference's kernel_test.py on CPU (with an empty stand-in for the compiled
`int4matmul` module, which that script imports at the top but which the helpers used here never
call) and records, for seeded inputs:
  * _pack_dense_weights_pow2 (kernel_test.py:60-80) for int4 and int2,
  * _pack_dense_weights_3   (kernel_test.py:82-123) for int3,
  * generate_dequantized_mtx (kernel_test.py:138-157): the fp16 weight W and the fp32 weight hiW,
  * the script's two comparators x @ W (fp16) and x.float() @ hiW (kernel_test.py:248-252).
The reference has no CPU code for the 16:32 sparse packer, the exponent coding or the kernels
themselves, so no vectors exist for those.
"""
import os
import sys
import types

import numpy as np
import torch


def main(ref_dir: str) -> None:
    sys.modules.setdefault("int4matmul", types.ModuleType("int4matmul"))
    sys.path.insert(0, ref_dir)
    import kernel_test as kt  # noqa: E402  (the reference's script; the __main__ part does not run)

    out_dir = os.path.dirname(os.path.abspath(__file__))
    gen = torch.Generator().manual_seed(20240611)

    cases = [  # bits, N, S, group
        (4, 128, 64, 64), (4, 256, 128, 128), (2, 128, 64, 64), (2, 256, 64, 128),
        (3, 128, 64, 64), (3, 256, 128, 128),
    ]
    blob = {}
    for bits, n, s, g in cases:
        tag = f"b{bits}_n{n}_s{s}_g{g}"
        q_sn = torch.randint(0, 1 << bits, (s, n), dtype=torch.int, generator=gen)
        if bits == 3:
            packed = kt._pack_dense_weights_3(q_sn.clone())
        else:
            packed = kt._pack_dense_weights_pow2(bits, q_sn.clone())
        n_groups = n // g
        zeros = torch.randint(0, 1 << bits, (n_groups, s), dtype=torch.int, generator=gen).to(torch.float16)
        scales = (torch.rand((n_groups, s), generator=gen) * 1.0 + 0.01).to(torch.float16)
        kt.GROUP_QUANTIZATION_SIZE = g
        w16, w32 = kt.generate_dequantized_mtx(q_sn.clone(), zeros, scales, n_groups)
        x = (torch.rand((1, 5, n), generator=gen) * 2.0 - 1.0).to(torch.float16)
        y16 = kt.fp16_fp16_matmul(w16.contiguous(), x)
        y32 = kt.fp32_fp32_matmul(w32.contiguous(), x)
        blob[tag + "_q_sn"] = q_sn.numpy().astype(np.uint8)
        blob[tag + "_packed"] = packed.numpy().astype(np.int32)
        blob[tag + "_zeros"] = zeros.numpy()
        blob[tag + "_scales"] = scales.numpy()
        blob[tag + "_w16"] = w16.contiguous().numpy()
        blob[tag + "_w32"] = w32.contiguous().numpy()
        blob[tag + "_x"] = x.numpy()
        blob[tag + "_y16"] = y16.numpy()
        blob[tag + "_y32"] = y32.numpy()
    np.savez_compressed(os.path.join(out_dir, "reference_python_vectors.npz"), **blob)
    print("wrote", len(blob), "arrays")


if __name__ == "__main__":
    if len(sys.argv) < 2 and not os.environ.get("INT4MATMUL_REFERENCE_DIR"):
        sys.exit("usage: make_golden.py /path/to/reference   (or set INT4MATMUL_REFERENCE_DIR)")
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["INT4MATMUL_REFERENCE_DIR"])
