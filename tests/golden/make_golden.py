"""Generate the golden fixtures in this folder from the reference's own code.

Run once, in a container that has the reference checked out (argument 1 or
``$RESET_REFERENCE``), with ``python tests/golden/make_golden.py <reference>``. It executes
the reference's CPU-runnable code on seeded inputs and stores inputs and
outputs as small ``.npz`` files; the tests then need neither the reference
nor this script. Nothing here is imported by the package or by ``bench.py``.

Sources of truth executed here:
* kernels/tests/conftest.py: ``_FP4_E2M1``, ``_fp8_e4m3_decode``,
  ``dequant_nvfp4``, ``reference_gemv``, ``random_nvfp4_tensor``.
* kernels/python/nvfp4r/vllm_integration.py: ``_unswizzle_blockscale`` (the one
  function is compiled out of the file's text, because importing the module
  needs the reference's built CUDA extension).
* reset/reset/logits_processor.py: ``ReSETRequest``, ``entropy_of``,
  ``scale_by_temperature``.
* the installed vLLM's CPU emulation of the activation quantizer
  (``ref_nvfp4_quant``) and its ``swizzle_blockscale`` - third-party stand-ins
  for the CUDA op the reference calls at vllm_integration.py:213.
"""

from __future__ import annotations

import ast
import hashlib
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path.insert(0, str(REPO))

from oracle import nvfp4 as onv  # noqa: E402  (input generators only)
from oracle import reset_policy as orp  # noqa: E402


def _load_reference(ref: Path):
    sys.path.insert(0, str(ref / "kernels" / "tests"))
    sys.path.insert(0, str(ref / "reset"))
    import conftest as ref_conftest  # type: ignore
    from reset import logits_processor as ref_lp  # type: ignore

    src = (ref / "kernels/python/nvfp4r/vllm_integration.py").read_text()
    tree = ast.parse(src)
    fn = next(n for n in tree.body
              if isinstance(n, ast.FunctionDef) and n.name == "_unswizzle_blockscale")
    ns: dict = {"torch": torch}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), "ref_unswizzle", "exec"), ns)
    return ref_conftest, ref_lp, ns["_unswizzle_blockscale"]


def make_decode_and_gemv(ref_conftest, out: Path):
    all_bytes = torch.arange(256, dtype=torch.uint8)
    e4m3 = ref_conftest._fp8_e4m3_decode(all_bytes).numpy()
    e2m1 = ref_conftest._FP4_E2M1.numpy()
    cases = {}
    for i, (L, N, K) in enumerate([(1, 64, 256), (2, 48, 512), (4, 32, 1024), (1, 8, 4096)]):
        w, ws = ref_conftest.random_nvfp4_tensor((1, N), K, device="cpu", seed=10 + i)
        w, ws = w.expand(L, N, K // 2), ws.expand(L, N, K // 16)
        x, xs = ref_conftest.random_nvfp4_tensor((L, 1), K, device="cpu", seed=20 + i)
        y = ref_conftest.reference_gemv(w, ws, x, xs)
        dq = ref_conftest.dequant_nvfp4(w[0, :4], ws[0, :4])
        cases[f"c{i}_w"] = w[0].contiguous().numpy()
        cases[f"c{i}_ws"] = ws[0].contiguous().numpy()
        cases[f"c{i}_x"] = x.numpy()
        cases[f"c{i}_xs"] = xs.numpy()
        cases[f"c{i}_y"] = y.numpy()
        cases[f"c{i}_dq4"] = dq.numpy()
    # full scale-byte range incl. large scales (fp32 result, no fp16 cast issue)
    w, ws = ref_conftest.random_nvfp4_tensor((1, 16), 256, device="cpu", seed=31,
                                             scale_max_byte=0x7F)
    cases["wide_w"], cases["wide_ws"] = w[0].numpy(), ws[0].numpy()
    cases["wide_dq"] = ref_conftest.dequant_nvfp4(w[0], ws[0]).numpy()
    np.savez_compressed(out / "nvfp4_decode_gemv.npz", e4m3_table=e4m3, e2m1_table=e2m1,
                        n_cases=np.int64(4), **cases)


def _values_to_codes(vals: torch.Tensor) -> np.ndarray:
    mags = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    idx = torch.bucketize(vals.abs().contiguous(), mags)
    assert torch.equal(mags[idx], vals.abs())
    return (idx | (torch.signbit(vals).long() << 3)).to(torch.uint8).numpy()


def make_quant(out: Path):
    from vllm.model_executor.layers.quantization.utils.nvfp4_emulation_utils import (
        ref_nvfp4_quant,
    )
    from vllm.model_executor.layers.quantization.utils.nvfp4_utils import swizzle_blockscale  # noqa: F401

    cases = {}
    shapes = [(1, 4096), (3, 512), (8, 1024), (2, 64)]
    for i, (M, K) in enumerate(shapes):
        g = torch.Generator().manual_seed(100 + i)
        x = torch.randn(M, K, generator=g, dtype=torch.float32)
        n_out = max(1, K // 1000)
        cols = torch.randperm(K, generator=g)[:n_out]
        x[:, cols] *= 20.0
        if i == 1:
            x[0, :32] = 0.0                       # all-zero blocks
            x[1, 32:48] = 1e-6                    # scale underflows to 0
            x[2, 64:80] = -0.0
        x = x.to(torch.bfloat16)
        amax = x.float().abs().max()
        gs = (amax / (6.0 * 448.0)).to(torch.float32)
        gs_inv = (1.0 / gs).to(torch.float32)
        vals, scale = ref_nvfp4_quant(x, gs_inv, 16)
        codes = _values_to_codes(vals.reshape(M, K))
        sf_bytes = scale.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        cases[f"q{i}_x_bf16"] = x.view(torch.int16).numpy().view(np.uint16)
        cases[f"q{i}_gs_inv"] = np.float32(gs_inv.item())
        cases[f"q{i}_codes"] = onv.pack_codes(codes)
        cases[f"q{i}_sf"] = sf_bytes
    np.savez_compressed(out / "quant_vllm_emulation.npz", n_cases=np.int64(len(shapes)), **cases)


def make_swizzle(ref_unswizzle, out: Path):
    cases = {}
    shapes = [(128, 64), (200, 320), (8, 4096), (130, 96)]
    for i, (M, K) in enumerate(shapes):
        rng = np.random.default_rng(200 + i)
        flat = rng.integers(0, 255, size=(M, K // 16), dtype=np.uint8)
        Mp, Cp = (M + 127) // 128 * 128, (K // 16 + 3) // 4 * 4
        sw = rng.integers(0, 255, size=(Mp, Cp), dtype=np.uint8)
        un = ref_unswizzle(torch.from_numpy(sw), M=M, K=K).numpy()
        cases[f"s{i}_flat"] = flat
        cases[f"s{i}_sw_in"] = sw
        cases[f"s{i}_unswizzled"] = un
        cases[f"s{i}_MK"] = np.array([M, K], dtype=np.int64)
    np.savez_compressed(out / "swizzle.npz", n_cases=np.int64(len(shapes)), **cases)


def make_reset(ref_lp, out: Path):
    cases = {}
    cfgs = [
        # (vocab, steps, seed, t_high, t_low, tau0, window, sigma)
        (512, 96, 7, 1.0, 0.1, 0.5505, 32, 3.0),
        (4096, 400, 8, 1.0, 0.1, 0.5505, 32, 3.0),
        (4096, 300, 9, 1.0, 0.3, 5.2, 8, 1.5),
        (151936, 48, 10, 1.0, 0.1, 0.5505, 32, 3.0),
        (4096, 64, 11, 1.0, 0.0, 6.0, 4, 2.0),     # t_low <= 1e-6: one-hot branch
    ]
    for i, (V, steps, seed, th, tl, tau0, w, sigma) in enumerate(cfgs):
        delim = V - 5
        nl = V - 9
        ids = orp.synthetic_token_stream(steps, delim, V, seed, gap_lo=10, gap_hi=30)
        if i == 2:                                 # exercise the two-newline rule
            ids[50:52] = nl
            ids[120] = nl
            ids[200:203] = nl
        req = ref_lp.ReSETRequest(th, tl, tau0, w, [nl], [delim])
        ents, temps, sums = [], [], []
        logits_all = orp.synthetic_logits(steps, V, seed, sigma=sigma)
        sha = hashlib.sha256(logits_all.numpy().tobytes()).hexdigest()
        for t in range(steps):
            row = logits_all[t]
            history = ids[:t].tolist()
            ent = ref_lp.entropy_of(row)
            scaled = req(history, row)
            ents.append(ent)
            ratio = None
            if torch.isinf(scaled).any():
                temps.append(0.0)
            else:
                j = int(torch.argmax(row.abs()))
                ratio = float(row[j] / scaled[j])
                temps.append(th if abs(ratio - th) < abs(ratio - tl) else tl)
            finite = torch.where(torch.isinf(scaled), torch.zeros_like(scaled), scaled)
            sums.append(float(finite.double().sum()))
        cases[f"r{i}_cfg"] = np.array([V, steps, seed, th, tl, tau0, w, sigma, delim, nl],
                                      dtype=np.float64)
        cases[f"r{i}_ids"] = ids
        cases[f"r{i}_entropy"] = np.array(ents, dtype=np.float64)
        cases[f"r{i}_temp"] = np.array(temps, dtype=np.float64)
        cases[f"r{i}_scaled_sum"] = np.array(sums, dtype=np.float64)
        cases[f"r{i}_logits_sha256"] = np.array(sha)
        if V == 512:
            cases[f"r{i}_logits"] = logits_all.numpy()
            cases[f"r{i}_scaled_last"] = scaled.numpy()
    np.savez_compressed(out / "reset_policy.npz", n_cases=np.int64(len(cfgs)), **cases)


def main():
    where = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("RESET_REFERENCE")
    if not where:
        sys.exit("usage: make_golden.py <path to the reference checkout>")
    ref = Path(where)
    ref_conftest, ref_lp, ref_unswizzle = _load_reference(ref)
    make_decode_and_gemv(ref_conftest, HERE)
    make_swizzle(ref_unswizzle, HERE)
    make_quant(HERE)
    make_reset(ref_lp, HERE)
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
