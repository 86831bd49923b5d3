"""Generate the golden vectors in this directory by RUNNING THE REFERENCE's own
Python code on CPU.  Needs a checkout of the reference (himikk/vllm-quant-kernels;
its path in $VQK_REFERENCE), torch, triton and vllm importable; no GPU.

    VQK_REFERENCE=<reference checkout> python tests/golden/make_golden.py

What runs:
  * the reference's torch quantizers and `_init_*` methods, unmodified, on CPU
    tensors (src/vllm_quant_kernels/_quant.py);
  * the reference's launchers `_int8_forward / _w8a8_forward / _fp8_forward`
    with its Triton kernels executed by the Triton interpreter
    (TRITON_INTERPRET=1); only the autotuner wrapper is bypassed because it
    needs a GPU driver, the kernel bodies are the reference's;
  * the reference's `fused_gumbel_sample` and `_compute_topk_threshold`
    (interpreter), plus a three-line Triton kernel calling `tl.rand` to pin the
    Philox stream;
  * vLLM's `apply_top_k_top_p_pytorch` on CPU for the top-p mask;
  * for MXFP8 / MXFP4 logits (`tl.dot_scaled` does not interpret): the
    reference quantizers + the dequantise-then-matmul reference from the
    reference's tests (tests/test_mxfp4_kernel.py:57-77).

Inputs are stored next to outputs, so the tests never depend on an RNG.
"""

import os
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"
REF = os.environ.get("VQK_REFERENCE")
if not REF or not os.path.isdir(os.path.join(REF, "src")):
    raise SystemExit("set VQK_REFERENCE to a checkout of the reference (the directory that holds src/ and tests/)")
sys.path.insert(0, os.path.join(REF, "src"))
sys.path.insert(0, os.path.join(REF, "tests"))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402
import triton.language as tl  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def save(name, **arrays):
    path = os.path.join(HERE, name)
    np.savez_compressed(path, **arrays)
    print(f"wrote {name}: " + ", ".join(f"{k}{tuple(v.shape)}" for k, v in arrays.items()))


class _FakeWeight:
    def __init__(self, t):
        self.data = t
        self.dtype = t.dtype
        self.shape = t.shape
        self.device = t.device


class _Shim:
    """Stands in for the Autotuner object: `shim[grid](*args, **kw)` runs the
    reference's jitted function in the interpreter with one fixed tile shape and
    records the positional arguments the launcher passed."""

    def __init__(self, kernel, **meta):
        self.fn = kernel.fn
        self.meta = meta
        self.calls = []

    def __getitem__(self, grid):
        def run(*args, **kw):
            self.calls.append(args)
            g = grid(self.meta) if callable(grid) else grid
            kw = dict(kw)
            kw.update(self.meta)
            return self.fn[g](*args, **kw)
        return run


def weight_matrix(rng, V, K, dtype=torch.float16):
    std = np.exp(rng.uniform(np.log(0.007), np.log(0.042), size=V)).astype(np.float32)
    w = rng.standard_normal((V, K), dtype=np.float32) * std[:, None]
    w = np.clip(w, -0.19, 0.19)
    t = torch.from_numpy(w).to(dtype)
    # edge rows
    t[0].zero_()                                   # all-zero row / groups
    t[1, :32] = torch.tensor([-0.0] * 32, dtype=dtype)   # a group of negative zeros
    t[2, 5] = 60000.0 if dtype == torch.float16 else 3.0e38   # huge outlier
    t[3] = t[3] * 1e-4                             # tiny values (fp16 subnormals)
    # E2M1 tie group: max 6 * 2^-5 so scale = 2^-5; midpoints are exact ties
    ties = [6.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0,
            -6.0, -0.1, 0.1, -0.0, 0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 5.5, 4.5, 0.3, 0.7, 2.4, 2.6]
    t[4, :32] = (torch.tensor(ties, dtype=torch.float32) * 2.0 ** -5).to(dtype)
    # e4m3 tie group: max 448 * 2^-12 so scale 2^-12; values at e4m3 midpoints
    t[5, :32] = (torch.linspace(-448, 448, 32) * 2.0 ** -12).to(dtype)
    return t


def main():
    from vllm_quant_kernels import _kernels as K
    from vllm_quant_kernels import _quant as RQ
    from vllm_quant_kernels import _sampler as RS
    from vllm_quant_kernels._sampler_kernels import fused_gumbel_sample

    rng = np.random.default_rng(20240611)

    # ---- A. exhaustive fp16 -> e4m3fn table (torch cast, _quant.py:60,308,413)
    allh = torch.arange(65536, dtype=torch.int32).to(torch.uint16).view(torch.float16)
    tab = allh.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    # same through fp32 (the weight path casts fp32 values)
    tab32 = allh.float().to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert (tab == tab32).all()
    save("e4m3_table_fp16.npz", table=tab)

    # ---- B. weight quantizers, reference code executed
    proc = RQ.QuantizedLogitsProcessor.__new__(RQ.QuantizedLogitsProcessor)
    for dtype, tag in ((torch.float16, "f16"), (torch.bfloat16, "bf16")):
        w = weight_matrix(rng, 48, 256, dtype)
        out = {"w_bits": w.view(torch.int16).numpy()}
        lm = types.SimpleNamespace(weight=_FakeWeight(w))
        proc._init_int8_weights(lm, w, sys, False)
        out["int8_q"] = lm._int8_w.numpy()
        out["int8_s_bits"] = lm._int8_scales.view(torch.int16).numpy()
        lm = types.SimpleNamespace(weight=_FakeWeight(w))
        try:
            proc._init_w8a8(lm, w, sys)
        except Exception as e:  # kernel factory needs a driver; state is already set
            print("  (_init_w8a8 kernel factory:", type(e).__name__, ")")
        out["w8a8_q"] = lm._w8a8_w.numpy()
        out["w8a8_s"] = lm._w8a8_scales.numpy()
        lm = types.SimpleNamespace(weight=_FakeWeight(w))
        try:
            proc._init_fp8(lm, w, sys)
        except Exception as e:
            print("  (_init_fp8 kernel factory:", type(e).__name__, ")")
        out["fp8_q"] = lm._fp8_w.numpy()
        out["fp8_s_bits"] = lm._fp8_scales.view(torch.int16).numpy()
        q, s = RQ._quantize_to_mxfp8(w)
        out["mxfp8_q"], out["mxfp8_s"] = q.numpy(), s.numpy()
        q, s = RQ._quantize_to_mxfp4(w)
        out["mxfp4_q"], out["mxfp4_s"] = q.numpy(), s.numpy()
        save(f"weight_quant_{tag}.npz", **out)

    # ---- C. launchers + Triton kernels in the interpreter
    V, Kd = 256, 128
    w = weight_matrix(rng, V, Kd)
    out = {"w_bits": w.view(torch.int16).numpy()}
    meta2 = dict(BLOCK_M=128, BLOCK_N=16, BLOCK_K=64)

    lm = types.SimpleNamespace(weight=_FakeWeight(w))
    proc._init_int8_weights(lm, w, sys, False)
    gmv_real = K.int8_gmv
    RQ.int8_gmv = _Shim(gmv_real, BLOCK_M=64, BLOCK_K=64)
    x1 = torch.from_numpy(rng.standard_normal((1, Kd), dtype=np.float32)).half()
    out["int8_x1_bits"] = x1.view(torch.int16).numpy()
    out["int8_logits1_bits"] = proc._int8_forward(x1, lm, None).view(torch.int16).numpy()
    gk, nb = K._make_thor_gemm_kernel()
    lm._int8_gemm_kernel, lm._int8_n_bucket = _Shim(gk, **meta2), nb
    x4 = torch.from_numpy(rng.standard_normal((4, Kd), dtype=np.float32)).half()
    bias = torch.from_numpy(rng.standard_normal(V, dtype=np.float32)).half()
    out["int8_x4_bits"] = x4.view(torch.int16).numpy()
    out["bias_bits"] = bias.view(torch.int16).numpy()
    out["int8_logits4_bits"] = proc._int8_forward(x4, lm, None).view(torch.int16).numpy()
    out["int8_logits4_bias_bits"] = proc._int8_forward(x4, lm, bias).view(torch.int16).numpy()
    RQ.int8_gmv = gmv_real

    lm = types.SimpleNamespace(weight=_FakeWeight(w))
    try:
        proc._init_w8a8(lm, w, sys)
    except Exception:
        pass
    gk, nb = K._make_thor_w8a8_gemm_kernel()
    shim = _Shim(gk, **meta2)
    lm._w8a8_gemm_kernel, lm._w8a8_n_bucket = shim, nb
    x3 = torch.from_numpy(rng.standard_normal((3, Kd), dtype=np.float32)).half()
    out["w8a8_x3_bits"] = x3.view(torch.int16).numpy()
    out["w8a8_logits3_bits"] = proc._w8a8_forward(x3, lm, None).view(torch.int16).numpy()
    out["w8a8_xq3"] = shim.calls[-1][2].numpy()                # xc passed to the kernel
    out["w8a8_xs3"] = np.float32(shim.calls[-1][4])            # x_scale.item()

    lm = types.SimpleNamespace(weight=_FakeWeight(w))
    try:
        proc._init_fp8(lm, w, sys)
    except Exception:
        pass
    gk, nb = K._make_thor_fp8_gemm_kernel()
    shim = _Shim(gk, **meta2)
    lm._fp8_gemm_kernel, lm._fp8_n_bucket = shim, nb
    x2 = torch.from_numpy(rng.standard_normal((2, Kd), dtype=np.float32) * 3).half()
    x2[0, 0] = 470.0     # > 464: the non-saturating cast gives NaN (byte 0x7f)
    x2[1, 1] = 464.0     # exactly the last value that still rounds to 448
    out["fp8_x2_bits"] = x2.view(torch.int16).numpy()
    out["fp8_logits2_bits"] = proc._fp8_forward(x2, lm, None).view(torch.int16).numpy()
    out["fp8_xq2"] = shim.calls[-1][2].view(torch.uint8).numpy()

    # ---- D. MX logits: reference quantizers + the reference tests' dequant matmul
    from test_mxfp4_accuracy import _dequantize_mxfp4
    x5 = torch.from_numpy(rng.standard_normal((5, Kd), dtype=np.float32)).half()
    out["mx_x5_bits"] = x5.view(torch.int16).numpy()
    xq, xs = RQ._quantize_to_mxfp8(x5)
    out["mx_xq5"], out["mx_xs5"] = xq.numpy(), xs.numpy()

    def deq8(v, s):
        R, Kk = v.shape
        return (v.view(torch.float8_e4m3fn).float().view(R, Kk // 32, 32)
                * torch.pow(2.0, s.float() - 127.0)[..., None]).view(R, Kk)

    wq8, ws8 = RQ._quantize_to_mxfp8(w)
    wq4, ws4 = RQ._quantize_to_mxfp4(w)
    out["mxfp8_logits5_bits"] = (deq8(xq, xs) @ deq8(wq8, ws8).t()).half().view(torch.int16).numpy()
    # tests/test_mxfp4_kernel.py:57-77 rounds both operands to fp16 before F.linear
    w4 = _dequantize_mxfp4(wq4, ws4)
    out["mxfp4_logits5_bits"] = (deq8(xq, xs) @ w4.t()).half().view(torch.int16).numpy()
    out["mxfp4_w_deq"] = w4.numpy()
    save("lm_head_forward.npz", **out)

    # ---- E. sampler (reference kernel in the interpreter)
    @triton.jit
    def _rand_kernel(out_ptr, seed_ptr, n, BLOCK: tl.constexpr):
        row = tl.program_id(0)
        offs = tl.program_id(1) * BLOCK + tl.arange(0, BLOCK)
        seed = tl.load(seed_ptr + row)
        u = tl.rand(seed, offs)
        tl.store(out_ptr + row * n + offs, u, mask=offs < n)

    seeds_r = torch.tensor([0, 1, 5, 123456, 2147483646, 42, -7], dtype=torch.int32)
    n = 4096
    u = torch.empty(len(seeds_r), n, dtype=torch.float32)
    _rand_kernel[(len(seeds_r), n // 1024)](u, seeds_r, n, BLOCK=1024)
    # far offsets too (global vocab indices of an 8-way shard)
    off2 = 248320 - 2048
    @triton.jit
    def _rand_kernel_off(out_ptr, seed_ptr, base, n, BLOCK: tl.constexpr):
        row = tl.program_id(0)
        offs = tl.program_id(1) * BLOCK + tl.arange(0, BLOCK)
        seed = tl.load(seed_ptr + row)
        u = tl.rand(seed, base + offs)
        tl.store(out_ptr + row * n + offs, u, mask=offs < n)
    u2 = torch.empty(len(seeds_r), 2048, dtype=torch.float32)
    _rand_kernel_off[(len(seeds_r), 2)](u2, seeds_r, off2, 2048, BLOCK=1024)
    save("philox_uniform.npz", seeds=seeds_r.numpy(), u=u.numpy(), base2=np.int64(off2), u2=u2.numpy())

    B, Vs = 8, 5000
    logits = torch.from_numpy(rng.standard_normal((B, Vs), dtype=np.float32) * 3)
    for i in range(B):
        logits[i, torch.from_numpy(rng.choice(Vs, 5, replace=False))] = 12.0
    logits[7, 100] = logits[7, 4000] = 15.0          # exact tie for the greedy row
    temp = torch.tensor([0.0, 1e-6, 0.5, 1.0, 1.5, 0.8, 1.2, 0.0], dtype=torch.float32)
    seeds = torch.tensor([3, 9, 11, 123456, 2147483000, 77, 31337, 1], dtype=torch.int32)
    res = {"logits": logits.numpy(), "temperature": temp.numpy(), "seeds": seeds.numpy()}
    res["tok_plain"] = fused_gumbel_sample(logits, temp, seeds).numpy()
    res["tok_notemp"] = fused_gumbel_sample(logits, None, seeds).numpy()
    for name, ks in (("k50", [50] * B), ("kmix", [1, 5, 50, 2, 50, 7, 3, 50])):
        top_k = torch.tensor(ks, dtype=torch.int32)
        thr = RS._compute_topk_threshold(logits, top_k, Vs)
        res[f"topk_{name}"] = top_k.numpy()
        res[f"thr_{name}"] = thr.numpy()
        res[f"tok_{name}"] = fused_gumbel_sample(logits, temp, seeds, topk_threshold=thr).numpy()
    assert RS._compute_topk_threshold(logits, torch.tensor([50] * 7 + [Vs], dtype=torch.int32), Vs) is None
    save("sampler_reference.npz", **res)

    # ---- F. top-p mask from vLLM (CPU)
    from vllm.v1.sample.ops.topk_topp_sampler import apply_top_k_top_p_pytorch
    Bp, Vp = 6, 3000
    lg = torch.from_numpy(rng.standard_normal((Bp, Vp), dtype=np.float32) * 3)
    for i in range(Bp):
        lg[i, torch.from_numpy(rng.choice(Vp, 5, replace=False))] = 12.0
    T = torch.tensor([0.5, 0.7, 1.0, 1.3, 1.5, 0.9], dtype=torch.float32)
    y = lg / T[:, None]
    k = torch.tensor([50, 50, 50, 10, Vp, Vp], dtype=torch.int64)
    p = torch.tensor([0.9, 0.5, 0.99, 0.9, 0.9, 0.3], dtype=torch.float32)
    masked = apply_top_k_top_p_pytorch(y.clone(), k, p)
    masked_p = apply_top_k_top_p_pytorch(y.clone(), None, p)
    masked_k = apply_top_k_top_p_pytorch(y.clone(), k, None)
    save("topp_vllm.npz", logits=lg.numpy(), temperature=T.numpy(), top_k=k.numpy(), top_p=p.numpy(),
         keep_kp=torch.isfinite(masked).numpy(), keep_p=torch.isfinite(masked_p).numpy(),
         keep_k=torch.isfinite(masked_k).numpy())


if __name__ == "__main__":
    main()
