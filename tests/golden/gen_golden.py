"""Generate the golden fixtures by running the compiled, unmodified reference on a Blackwell GPU.

    bash oracle/build_ref.sh                      # where the reference sources are mounted
    python tests/golden/gen_golden.py [outdir]    # on a B200; default outdir = tests/golden

For every case of ``cases.py`` the reference extension (oracle/_ref/mxdsa_ext.so) is called
through its own public entry points and the outputs are stored as ``<case>.npz``:

  input_hash         sha256 of the input tensors (the tests rebuild them from the seed and compare)
  out_rows, out_kept bf16 bit patterns (uint16) of the kept (token, head) rows and their indices
  out_sum, out_abs   float64 sum and sum of magnitudes over the 512 dims of EVERY (token, head) row
  max_logits, lse    complete float32 outputs
  sched_meta, num_splits, num_sm_parts   (decode) what the reference's scheduler produced

``probes.npz`` holds four tiny single-purpose runs that pin how the kernel pairs Q bytes with K
bytes, which scale byte it applies to which block, which w1/w2 word scales which output
dimensions, and which index row a decode query follows.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, "..", ".."))
sys.path.insert(0, HERE)
import cases  # noqa: E402
from oracle import mxdsa_oracle as O  # noqa: E402


def load_reference():
    path = os.path.join(ROOT, "oracle", "_ref", "mxdsa_ext.so")
    spec = importlib.util.spec_from_file_location("mxdsa_ext", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _t(x, dev="cuda"):
    return None if x is None else torch.from_numpy(np.ascontiguousarray(x)).to(dev)


def run_prefill(ext, c):
    out, mxl, lse = ext.dual_mxfp8_head64_sparse_prefill_fwd(
        _t(c["q"]), _t(c["kv"]), _t(c["indices"]), c["sm_scale"], c["w1"], c["w2"],
        _t(c["attn_sink"]), _t(c["topk_length"]))
    torch.cuda.synchronize()
    return out, mxl, lse


def run_decode(ext, c, meta=None, splits=None):
    out, lse, meta, splits = ext.dual_mxfp8_sparse_decode_fwd(
        _t(c["q"]), _t(c["kv"]), _t(c["indices"]), _t(c["topk_length"]), _t(c["attn_sink"]),
        meta, splits, _t(c["extra_kv"]), _t(c["extra_indices"]), _t(c["extra_topk_length"]),
        512, 512, c["sm_scale"], c["w1"], c["w2"])
    torch.cuda.synchronize()
    return out, lse, meta, splits


def summarise_out(out: torch.Tensor) -> dict:
    rows = out.reshape(-1, 512)
    kept = cases.kept_rows(rows.shape[0])
    f = rows.double()
    return dict(out_kept=kept,
                out_rows=rows[torch.from_numpy(kept).to(rows.device)].view(torch.int16).cpu().numpy().view(np.uint16),
                out_sum=f.sum(-1).cpu().numpy(), out_abs=f.abs().sum(-1).cpu().numpy())


def probes(ext) -> dict:
    """Single-purpose runs; every value written is exactly representable so the answers are exact."""
    res = {}
    one = 0x38  # E4M3 1.0
    w_one = [0x7F7F7F7F] * 8

    def q_rows(n_tok):
        q = np.zeros((n_tok, 64, 528), dtype=np.uint8)
        q[..., 512:] = 127
        return q

    def kv_rows(n):
        data = np.zeros((n, 512), dtype=np.uint8)
        slots = np.full((n, 16), 127, dtype=np.uint8)
        return data, slots

    def pack(data, slots):
        n = data.shape[0]
        return np.concatenate([data.reshape(-1), slots.reshape(-1)]).reshape(n, 1, 528)

    # (i) pairing: pair m has Q memory block m = 1.0; token k has K block k = 1.0 (V too).
    q = q_rows(32)
    for m in range(16):
        q[2 * m:2 * m + 2, :, 32 * m:32 * m + 32] = one
    data, slots = kv_rows(64)
    for k in range(16):
        data[k, 32 * k:32 * k + 32] = one
    idx = np.full((16, 1, 64), -1, dtype=np.int32)
    idx[:, 0, :16] = np.arange(16)
    out, mxl, lse = ext.dual_mxfp8_head64_sparse_prefill_fwd(
        _t(q), _t(pack(data, slots)), _t(idx), 1.0, w_one, w_one, None, None)
    res["pair_out"] = out.float().cpu().numpy()[::2, 0, ::32]      # [16 pairs, 16 blocks]
    res["pair_max"] = mxl.cpu().numpy()[::2, 0]

    # (ii) scale bytes: pair m attends token m only.  Q: all ones, scale byte g = 127+g+1.
    q = q_rows(32)
    q[..., :512] = one
    q[..., 512:520] = 127 + 1 + np.arange(8)
    q[..., 520:528] = 127 + 1 + np.arange(8)
    idx = np.full((16, 1, 64), -1, dtype=np.int32)
    idx[:, 0, 0] = np.arange(16)
    out, mxl, lse = ext.dual_mxfp8_head64_sparse_prefill_fwd(
        _t(q), _t(pack(data, slots)), _t(idx), 1.0, w_one, w_one, None, None)
    res["qscale_logit"] = mxl.cpu().numpy()[::2, 0]                # 32 * 2^(q scale used for K block m)
    #      K: token k block k ones, K scale byte j = 127+j+1; Q scales 1.
    q = q_rows(32)
    q[..., :512] = one
    slots2 = slots.copy()
    slots2[:, :8] = 127 + 1 + np.arange(8)
    slots2[:, 8:] = 127 + 1 + np.arange(8)
    out, mxl, lse = ext.dual_mxfp8_head64_sparse_prefill_fwd(
        _t(q), _t(pack(data, slots2)), _t(idx), 1.0, w_one, w_one, None, None)
    res["kscale_logit"] = mxl.cpu().numpy()[::2, 0]
    res["kscale_out"] = out.float().cpu().numpy()[::2, 0, ::32]    # V value of token m's block m

    # (iii) w words: one token of all ones, w1 word j byte = 127+j, w2 word j byte = 117+j.
    data3, slots3 = kv_rows(64)
    data3[0] = one
    idx = np.full((1, 1, 64), -1, dtype=np.int32)
    idx[0, 0, 0] = 0
    q = q_rows(2)
    q[..., :512] = one
    w1 = [int((127 + j) * 0x01010101) for j in range(8)]
    w2 = [int((117 + j) * 0x01010101) for j in range(8)]
    out, _, _ = ext.dual_mxfp8_head64_sparse_prefill_fwd(
        _t(q), _t(pack(data3, slots3)), _t(idx), 1.0, w1, w2, None, None)
    res["w_out"] = out.float().cpu().numpy()[0, 0]                 # [512]
    #      distinct bytes inside one word: which byte is applied at which token position
    w1b = [0x7F807F80 if j == 0 else 0x7F7F7F7F for j in range(8)]
    idx = np.full((4, 1, 128), -1, dtype=np.int32)
    for p, pos in enumerate((0, 32, 64, 96)):
        idx[p, 0, pos] = 0
    q = q_rows(8)
    q[..., :512] = one
    out, _, _ = ext.dual_mxfp8_head64_sparse_prefill_fwd(
        _t(q), _t(pack(data3, slots3)), _t(idx), 1.0, w1b, w_one, None, None)
    res["w_byte_out"] = out.float().cpu().numpy()[::2, 0, 0]       # [4 positions]

    # (iv) decode index rows: 4 queries, row r points at token r whose values are all (r+1)/8...
    pool = np.zeros((2, 64, 528), dtype=np.uint8)
    flat = pool.reshape(2, -1)
    codes = [0x28, 0x30, 0x38, 0x40, 0x44, 0x48]                   # 0.25 0.5 1 2 3 4
    for r in range(6):
        flat[0, r * 512:(r + 1) * 512] = codes[r]
    flat[:, 64 * 512:] = 127
    qd = np.zeros((1, 6, 64, 528), dtype=np.uint8)
    qd[..., :512] = one
    qd[..., 512:] = 127
    idx = np.full((1, 6, 64), -1, dtype=np.int32)
    idx[0, :, 0] = np.arange(6)
    out, lse, meta, splits = ext.dual_mxfp8_sparse_decode_fwd(
        _t(qd), _t(pool.reshape(2, 64, 1, 528)), _t(idx), None, None, None, None, None, None, None,
        512, 512, 1.0, w_one, w_one)
    torch.cuda.synchronize()
    res["decode_row_out"] = out.float().cpu().numpy()[0, :, 0, 0]  # value each query saw
    res["decode_lse_shape"] = np.array(lse.shape)
    res["decode_lse_stride"] = np.array(lse.stride())
    return res


def main():
    outdir = sys.argv[1] if len(sys.argv) > 1 else HERE
    os.makedirs(outdir, exist_ok=True)
    ext = load_reference()
    props = torch.cuda.get_device_properties(0)
    print("device", props.name, props.major, props.minor, props.multi_processor_count, flush=True)
    np.savez_compressed(os.path.join(outdir, "probes.npz"), **probes(ext))
    print("probes done", flush=True)
    for name in cases.PREFILL_CASES:
        c = cases.build(name)
        out, mxl, lse = run_prefill(ext, c)
        np.savez_compressed(os.path.join(outdir, name + ".npz"), input_hash=cases.input_hash(c),
                            max_logits=mxl.cpu().numpy(), lse=lse.cpu().numpy(), **summarise_out(out))
        print("golden", name, tuple(out.shape), flush=True)
    for name in cases.DECODE_CASES:
        c = cases.build(name)
        out, lse, meta, splits = run_decode(ext, c)
        # a second call that reuses the returned scheduling info must give the same answer
        out2, lse2, _, _ = run_decode(ext, c, meta, splits)
        assert torch.equal(out.view(torch.int16), out2.view(torch.int16))
        np.savez_compressed(os.path.join(outdir, name + ".npz"), input_hash=cases.input_hash(c),
                            lse=lse.contiguous().cpu().numpy(), lse_shape=np.array(lse.shape),
                            sched_meta=meta.cpu().numpy(), num_splits=splits.cpu().numpy(),
                            num_sm_parts=meta.shape[0], sm_count=props.multi_processor_count,
                            **summarise_out(out))
        print("golden", name, tuple(out.shape), flush=True)
    # scheduler-only goldens at the benchmark shapes (tiny pools: every index points at page 0)
    sched = {}
    for b in (64, 128):
        for extra in (0, 128, 1024, 4096):
            q = torch.zeros(b, 6, 64, 528, dtype=torch.uint8, device="cuda")
            q[..., 512:] = 127
            pool = torch.zeros(2, 64, 1, 528, dtype=torch.uint8, device="cuda")
            idx = torch.zeros(b, 6, 128, dtype=torch.int32, device="cuda")
            eidx = torch.zeros(b, 6, extra, dtype=torch.int32, device="cuda") if extra else None
            _, _, meta, splits = ext.dual_mxfp8_sparse_decode_fwd(
                q, pool, idx, None, None, None, None, pool if extra else None, eidx, None,
                512, 512, 1.0, [0x7F7F7F7F] * 8, [0x7F7F7F7F] * 8)
            torch.cuda.synchronize()
            sched[f"meta_b{b}_e{extra}"] = meta.cpu().numpy()
            sched[f"splits_b{b}_e{extra}"] = splits.cpu().numpy()
    np.savez_compressed(os.path.join(outdir, "sched.npz"), **sched)
    print("golden sched done", flush=True)


if __name__ == "__main__":
    main()
