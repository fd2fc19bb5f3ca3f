"""Generate tests/golden/callers_gen1_ref.txt, callers_gen2_ref.txt and callers_gen2_ref_scalar.txt: the output of
tests/cpp/callers_program.cpp built against the REFERENCE ITSELF (oracle/build_callers_ref.sh
builds oracle/_ref/callers_gen{1,2}_ref from the reference's own sources first) — and
verify_gen1_ref.txt: what the reference's own root verify.cpp prints when linked with the reference.

    oracle/build_callers_ref.sh <reference root> && python tests/golden/make_callers_golden.py

The GPU builds of the same program (tests/cpp/build_callers.sh: the reference's autograd.cpp,
layer.cpp and loss.cpp unchanged over the B200 host layers) are compared with these lines on
machines that have no reference.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def main():
    for name in ("callers_gen1_ref", "callers_gen2_ref", "callers_gen2_ref_scalar", "verify_gen1_ref"):
        exe = os.path.join(ROOT, "oracle", "_ref", name)
        out = subprocess.run([exe], capture_output=True, text=True, check=True, cwd="/tmp").stdout
        path = os.path.join(HERE, f"{name}.txt")
        with open(path, "w") as f:
            f.write(out)
        print(f"wrote {len(out.splitlines())} lines -> {path}")


if __name__ == "__main__":
    main()
