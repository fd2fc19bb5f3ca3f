"""Generate tests/golden/golden_cases.npz from the REAL reference.

Run where the reference sources exist (oracle/build_ref.sh builds oracle/_ref/ first):

    python tests/golden/make_golden.py

For every case of tests/cases.py the file stores the input storage buffers with their view
metadata and the output the compiled reference produced (a SHA-256 digest of it for the
bit-exact cases, the values themselves where a tolerance applies) (the back-end named by the case:
scalar/OpenMP `*_mp`, or the AVX2 / AVX-512 SIMD functions for the fp32 transcendental
flavours).  The tests then check the plain-C oracle and the CUDA path against these vectors
on machines that have no reference.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import cases as C          # noqa: E402
import oracle_lib as ol    # noqa: E402


def main():
    ref = ol.Reference()
    assert ref.has_avx2 and ref.has_avx512, "golden generation needs an AVX2+AVX-512 host"
    out = {}
    names = []
    for case in C.all_cases():
        n = case["name"]
        assert n not in names, n
        names.append(n)
        for i, v in enumerate(case["views"]):
            key = C.digest(v.buf)[:16]                 # each distinct storage buffer is stored once
            out["buf/" + key] = v.buf
            out[f"{n}/in{i}/key"] = np.array(key)
            out[f"{n}/in{i}/meta"] = np.array([v.offset, len(v.shape), *v.shape, *v.strides], np.int64)
        res = C.run_case(ref, case)
        if case["exact"]:
            out[f"{n}/digest"] = np.array(C.digest(res))   # bit-exact cases: a digest is enough
        else:
            out[f"{n}/out"] = res
    out["__names__"] = np.array(names)
    path = os.path.join(HERE, "golden_cases.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {len(names)} cases, {os.path.getsize(path) / 1024:.0f} KiB -> {path}")


if __name__ == "__main__":
    main()
