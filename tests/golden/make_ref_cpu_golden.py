"""Writes tests/golden/ref_cpu_golden.npz: outputs of the reference project's own CPU kernels
(oracle/_ref/libref_cpu.so and libref_cpu_seq.so, built by `make -C oracle ref REF=<checkout>`)
on the seeded cases of tests/refcpu.py.  Keys are `<build>/<case>.<output>` with build `arma`
(reductions as Armadillo's own loops run them) or `seq` (plain index order).

    python tests/golden/make_ref_cpu_golden.py
"""
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from tests import refcpu  # noqa: E402


def main():
    data = {}
    for build, seq in (("arma", False), ("seq", True)):
        impl = refcpu.load(seq)
        if impl is None:
            raise SystemExit("oracle/_ref/libref_cpu*.so missing: run `make -C oracle ref REF=<reference checkout>`")
        assert impl.sequential == seq
        for key, val in refcpu.run_all(impl).items():
            data[f"{build}/{key}"] = val
    np.savez_compressed(refcpu.GOLDEN, **data)
    print("wrote", refcpu.GOLDEN, sum(v.nbytes for v in data.values()), "bytes of arrays")


if __name__ == "__main__":
    main()
