"""Generate the golden vectors under tests/golden/ by running the REFERENCE's own code.

Needs the reference tree (not present on the GPU box) and oracle/_ref/fr_ref_run, which
oracle/build_ref.py builds from the reference's model.cpp + kernels/default/* + kernels/cpu/* and the fp32
CPU primitives of oracle/ref/cpu_prims.cpp.  For each seeded tiny model the script writes the `.fr` file to
a temporary directory, runs `fr_ref_run <file> "cpu fp32"` on a seeded id sequence and stores
{shape name, seed, ids, logits of every step (float32)} in tests/golden/<name>.npz.  The committed .npz files
are what the tests read; this script is only re-run when the fixtures have to change.

  python tests/golden/make_golden.py
"""
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

CASES = [("tiny4", 101, 8), ("tiny4b", 102, 6), ("tiny50", 103, 6), ("tiny51", 104, 6), ("tiny52", 105, 6)]


def main():
    pkg = entry.load_package()
    synth = pkg.synth
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import build_ref
    exe = build_ref.build()
    with tempfile.TemporaryDirectory() as tmp:
        for name, seed, n in CASES:
            shape = synth.SHAPES[name]
            # weights on the fp16 grid, so that the same model can also be given to the "cuda fp16" strategy exactly
            _, tensors = synth.fp16_exact_pair(shape, synth.generate(shape, seed=seed, ln_random=True))
            fr = os.path.join(tmp, name + ".fr")
            synth.write_fr(fr, shape, tensors)
            ids = synth.token_ids(shape, n, seed=seed)
            out = os.path.join(tmp, name + ".bin")
            subprocess.check_call([exe, fr, "cpu fp32", out] + [str(int(i)) for i in ids])
            logits = np.fromfile(out, np.float32).reshape(n, shape.vocab)
            # seq mode of the reference = the same token loop (kernels/default/model_forward_seq.cpp:34-46)
            subprocess.check_call([exe, fr, "cpu fp32", out, "--seq"] + [str(int(i)) for i in ids])
            seq_last = np.fromfile(out, np.float32)
            assert np.array_equal(seq_last, logits[-1]), "reference seq mode differs from its token loop"
            np.savez_compressed(os.path.join(HERE, name + ".npz"), name=name, seed=seed, ids=ids, logits=logits)
            print(name, logits.shape, float(np.abs(logits).max()))


if __name__ == "__main__":
    main()
