"""Writes packers.npz: the bytes that the REFERENCE's own packers (tests/mxfp8_test_utils.py of the reference
tree, imported unmodified) produce for the seeded inputs of packer_cases.py.

    python tests/golden/gen_packer_golden.py <path of the reference checkout>

Runs on the CPU.  The fixture pins the wire format of this repository's three packers (torch, numpy oracle,
CUDA kernels) to the reference's.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import packer_cases as PC  # noqa: E402


def main():
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    path = os.path.join(sys.argv[1], "tests", "mxfp8_test_utils.py")
    spec = importlib.util.spec_from_file_location("reference_mxfp8_test_utils", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    out = {}
    for dtype in (torch.float32, torch.bfloat16):   # the inputs are bf16-exact: both dtypes must pack to the same bytes
        q = torch.from_numpy(PC.q_input()).to(dtype)
        kv = torch.from_numpy(PC.prefill_kv_input()).to(dtype)
        pages = torch.from_numpy(PC.decode_kv_input()).to(dtype)
        got = {"q": ref.pack_dual_q64(q)[0].numpy(), "prefill_kv": ref.pack_dual_prefill_kv64(kv)[0].numpy(),
               "decode_kv": ref.pack_dual_decode_kv_pages(pages)[0].numpy()}
        for k, v in got.items():
            assert k not in out or np.array_equal(out[k], v), k
            out[k] = v
    out["torch_version"] = np.array(torch.__version__)
    np.savez_compressed(os.path.join(HERE, "packers.npz"), **out)
    for k, v in out.items():
        print(k, getattr(v, "shape", ""), getattr(v, "dtype", ""))


if __name__ == "__main__":
    main()
