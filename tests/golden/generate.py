"""Regenerates the golden fixtures in this folder.  Needs a GPU and the reference sources.

    make -C oracle ref REF=/path/to/SpTMM        # builds oracle/_ref/ref_harness (unmodified reference kernels)
    python tests/golden/generate.py [outdir]     # default: this folder

The harness runs the reference's own prepareW_map and SpTMM kernels on seeded int8 activations
and writes, per case, X and C in full, every encoded array in full for the small cases, and an
FNV-1a checksum of every array in manifest.json.  reference_timing.jsonl records the reference
kernels' time per call on the GPU that produced the fixtures.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))

if __name__ == "__main__":
    out = sys.argv[1] if len(sys.argv) > 1 else HERE
    harness = os.path.join(ROOT, "oracle", "_ref", "ref_harness")
    if not os.path.exists(harness):
        raise SystemExit("build the harness first: make -C oracle ref REF=<reference checkout>")
    subprocess.run([harness, "dump", out], check=True)
