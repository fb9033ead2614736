"""Copies the reference's own golden dequantisation vectors into tests/golden/reference_data/.

The files are data, not source: raw ggml blocks (`*.raw`) and the f32 values llama-prism's
ggml produced from them (`*.f32`), kept by the reference under tests/data/ and used by its
tests/dequant_vs_ggml.rs.  They pin the oracle's weight decode bit-exactly.

    python tests/golden/import_reference_fixtures.py /path/to/reference
"""
import os
import shutil
import sys

NAMES = ["attn_k3", "ssm_out4", "attn_k3.ptq1", "ssm_out4.ptq1", "mtp_q80_3", "mtp_q6k3", "mtp_q4k3"]


def main(ref):
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_data")
    os.makedirs(dst, exist_ok=True)
    for n in NAMES:
        for ext in (".raw", ".f32"):
            shutil.copyfile(os.path.join(ref, "tests", "data", n + ext), os.path.join(dst, n + ext))
    print("copied", 2 * len(NAMES), "files to", dst)


if __name__ == "__main__":
    main(sys.argv[1])
