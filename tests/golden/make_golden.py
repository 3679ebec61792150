"""Generates tests/golden/matmul_family.json.

An independent restatement (pure-Python integers + numpy float32 scalars, one rounded
multiply and one rounded add per term) of FastNN's CPU matmul family, run on the fixture
inputs of FastNN's own tests:

* generator: SplitMix64 -> uniform [-1,1)          (tests/cuda_parity.rs:29-43)
* shapes and seeds: the six matmul-family cases      (tests/cuda_parity.rs:116-166,
                                                       tests/gradcheck.rs:277-331)
* arithmetic: i, p, j loop with `result += a*b`      (src/tensor/ops.rs:366-377,406-422),
  NT/TN as transpose-copy + NN                        (src/tensor/ops.rs:476-477,516-517)
* gradients: dA = dC.B^T (NT), dB = A^T.dC (TN)       (src/autograd/backward_ops.rs:82-134)
  with the upstream weights seeded 0xBADC0DE ^ len(name) (tests/cuda_parity.rs:74)

It deliberately shares no code with oracle/: the C oracle must reproduce these bit patterns.
Also stores the first SplitMix64 outputs, which can be checked against the published
SplitMix64 sequence (seed 0 -> 0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F).

Run:  python tests/golden/make_golden.py
"""
import json
import os

import numpy as np

MASK = (1 << 64) - 1
GOLD = 0x9E3779B97F4A7C15


def splitmix_stream(seed, n):
    s = (seed + GOLD) & MASK              # Rng::new
    out = []
    for _ in range(n):
        s = (s + GOLD) & MASK
        z = s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
        out.append(z ^ (z >> 31))
    return out


def rand_data(n, seed):
    f = np.float32
    return np.array([f(f(f(z >> 40) / f(1 << 24)) * f(2.0)) - f(1.0) for z in splitmix_stream(seed, n)],
                    dtype=np.float32)


def mm(a, b):
    """i-p-j nest, float32 multiply then float32 add."""
    m, k = a.shape
    n = b.shape[1]
    c = np.zeros((m, n), dtype=np.float32)
    for i in range(m):
        for p in range(k):
            av = a[i, p]
            for j in range(n):
                c[i, j] = np.float32(c[i, j] + np.float32(av * b[p, j]))
    return c


def bmm(a, b):
    return np.stack([mm(a[i], b[i]) for i in range(a.shape[0])])


def T(x):
    return np.ascontiguousarray(np.swapaxes(x, -1, -2))


def bits(x):
    return [int(v) for v in np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).ravel()]


CASES = [
    # name (as in cuda_parity.rs), op, a shape, b shape
    ("matmul_2d", "nn", (3, 4), (4, 5)),
    ("matmul_nt_2d", "nt", (3, 4), (5, 4)),
    ("matmul_tn_2d", "tn", (3, 4), (3, 5)),
    ("matmul_batched", "nn", (2, 3, 4), (2, 4, 5)),
    ("matmul_nt_batch", "nt", (2, 3, 4), (2, 5, 4)),
    ("matmul_tn_batch", "tn", (2, 4, 3), (2, 4, 5)),
]


def forward(op, a, b):
    f = mm if a.ndim == 2 else bmm
    if op == "nn":
        return f(a, b)
    if op == "nt":
        return f(a, T(b))
    return f(T(a), b)


def main():
    out = {"splitmix_seed0_reference_stream": [hex(v) for v in splitmix_stream(0, 3)], "cases": []}
    for name, op, sa, sb in CASES:
        a = rand_data(int(np.prod(sa)), 1).reshape(sa)
        b = rand_data(int(np.prod(sb)), 2).reshape(sb)
        c = forward(op, a, b)
        w = rand_data(c.size, 0xBADC0DE ^ len(name)).reshape(c.shape)     # upstream gradient
        f = mm if a.ndim == 2 else bmm
        # gradients of sum(c * w) w.r.t. the stored operands, through the reference's GradFns
        if op == "nn":      # dA = dC.B^T ; dB = A^T.dC
            ga, gb = f(w, T(b)), f(T(a), w)
        elif op == "nt":    # c = a.b^T : dA = dC.b ; db = dC^T.a
            ga, gb = f(w, b), f(T(w), a)
        else:               # c = a^T.b : da = b.dC^T ; db = a.dC
            ga, gb = f(b, T(w)), f(a, w)
        out["cases"].append({
            "name": name, "op": op, "a_shape": list(sa), "b_shape": list(sb),
            "a_bits": bits(a), "b_bits": bits(b), "c_shape": list(c.shape), "c_bits": bits(c),
            "w_bits": bits(w), "grad_a_bits": bits(ga), "grad_b_bits": bits(gb),
        })
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "matmul_family.json")
    with open(path, "w") as fh:
        json.dump(out, fh, indent=1)
    print("wrote", path)


if __name__ == "__main__":
    main()
