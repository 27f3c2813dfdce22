"""Generates tests/golden/metal_shader_vectors.npz.

Runs the reference's own Metal shader source (compiled as host C++ by
``oracle/Makefile`` into ``oracle/_ref``) on small seeded inputs and stores inputs
and outputs, so that the CPU restatement and the CUDA path can be checked against
the reference's arithmetic on machines where the reference tree is absent.

Run from the repository root, with the reference checkout available to the
Makefile:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402


def main():
    oracle.build()
    m = oracle.MetalRef()
    rng = np.random.default_rng(20261125)
    out = {}
    # batch distance matrices, all four metrics, odd sizes
    q = rng.standard_normal((7, 37)).astype(np.float32)
    x = rng.standard_normal((61, 37)).astype(np.float32)
    out["dist_q"], out["dist_x"] = q, x
    for mid, name in enumerate(["euclidean", "cosine", "dotProduct", "manhattan"]):
        out[f"dist_{name}"] = m.batch_distances(mid, q, x)
    # one query against N, d = 512 (the reference's specialised dimension)
    q1 = rng.uniform(-1, 1, 512).astype(np.float32)
    x1 = rng.uniform(-1, 1, (33, 512)).astype(np.float32)
    out["single_q"], out["single_x"] = q1, x1
    for mid, name in enumerate(["euclidean", "cosine", "dotProduct", "manhattan"]):
        out[f"single_{name}"] = m.distances(mid, q1, x1)
    # three Lloyd steps with the shader kernels; cluster 5 starts far away and stays empty
    kx = rng.standard_normal((300, 8)).astype(np.float32)
    c0 = kx[:6].copy()
    c0[5] = 1000.0
    out["km_x"], out["km_c0"] = kx, c0
    c = c0
    for it in range(3):
        c, asg, dist = m.kmeans_step(kx, c)
        out[f"km_c{it + 1}"], out[f"km_assign{it + 1}"], out[f"km_dist{it + 1}"] = c, asg, dist
    out["km_min_dist_sq"] = m.min_distances(kx, c0)
    # shader uint8 quantiser round trip
    v = rng.uniform(0, 1, 257).astype(np.float32)
    out["q_in"] = v
    out["q_codes"] = m.scalar_quantize(v, 255.0, 0.0)
    out["q_back"] = m.scalar_dequantize(out["q_codes"], 255.0, 0.0)
    # product quantisation shaders (productQuantize / productDequantize): 4 sub-spaces of 6 dimensions, 256
    # codewords; codeword 200 duplicates codeword 17 in every sub-space (a tie: the lower code must win) and the
    # first rows sit exactly on codewords
    px = rng.standard_normal((200, 24)).astype(np.float32)
    pcb = rng.standard_normal((4, 256, 6)).astype(np.float32)
    pcb[:, 200] = pcb[:, 17]
    for r in range(8):
        px[r] = np.concatenate([pcb[s, (17, 200, 3, 255)[(r + s) % 4]] for s in range(4)])
    out["pq_x"], out["pq_cb"] = px, pcb
    out["pq_codes"] = m.product_quantize(px, pcb)
    out["pq_back"] = m.product_dequantize(out["pq_codes"], pcb)
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "metal_shader_vectors.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
