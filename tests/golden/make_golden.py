"""Generates the golden fixtures in this directory.  Run once, in the build container:

    python tests/golden/make_golden.py [/path/to/reference]

Two independent sources pin the oracle:

1. ``cvt_tables.npz`` - the CUDA toolkit's HOST implementations of
   ``__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3)`` and
   ``__nv_cvt_float_to_fp6(x, __NV_E3M2, cudaRoundNearest)`` (cuda_fp8.h /
   cuda_fp6.h, the calls the reference quantizer makes at
   csrc/quantization.cu:58-67), tabulated for all 65536 bf16 bit patterns.  A
   tiny program is compiled with nvcc and run on the CPU.
2. ``reference_helpers.npz`` - outputs of the reference's own pure-torch test
   helpers (tests/test_ops.py: decode_e3m2, decode_ue8m0, cpu_pack_fp6,
   reference_gemm and the decode_mxfp8 procedure) imported from the read-only
   reference checkout, on seeded CPU inputs that are stored next to them.

The fixtures travel with the repository; the reference checkout does not.
"""

from __future__ import annotations

import importlib.util
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
sys.path.insert(0, str(ROOT))

CVT_SOURCE = r"""
#include <cuda_fp8.h>
#include <cuda_fp6.h>
#include <cstdio>
#include <cstdint>
#include <cstring>
int main() {
  for (uint32_t i = 0; i < 65536; ++i) {
    uint32_t bits = i << 16;
    float f;
    std::memcpy(&f, &bits, 4);
    unsigned char e4m3 = __nv_cvt_float_to_fp8(f, __NV_SATFINITE, __NV_E4M3);
    unsigned char e3m2 = __nv_cvt_float_to_fp6(f, __NV_E3M2, cudaRoundNearest);
    std::fputc(e4m3, stdout);
    std::fputc(e3m2, stdout);
  }
  return 0;
}
"""


def make_cvt_tables() -> None:
    with tempfile.TemporaryDirectory() as tmp:
        src = Path(tmp) / "cvt.cu"
        exe = Path(tmp) / "cvt"
        src.write_text(CVT_SOURCE)
        subprocess.run(["nvcc", "-O1", "-o", str(exe), str(src)], check=True)
        raw = subprocess.run([str(exe)], check=True, capture_output=True).stdout
    table = np.frombuffer(raw, dtype=np.uint8).reshape(65536, 2)
    np.savez_compressed(HERE / "cvt_tables.npz", e4m3=table[:, 0].copy(), e3m2=table[:, 1].copy())


def load_reference_helpers(reference_root: Path):
    spec = importlib.util.spec_from_file_location(
        "reference_test_ops", reference_root / "tests" / "test_ops.py"
    )
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def make_reference_fixtures(reference_root: Path) -> None:
    from oracle import mx_oracle as oracle

    ref = load_reference_helpers(reference_root)
    out: dict[str, np.ndarray] = {}

    # All 64 E3M2 codes and all 256 UE8M0 codes through the reference decoders.
    out["e3m2_table"] = ref.decode_e3m2(torch.arange(64, dtype=torch.uint8)).numpy()
    ue = ref.decode_ue8m0(torch.arange(256, dtype=torch.uint8))
    out["ue8m0_table_bits"] = ue.view(torch.int32).numpy()

    # Bitstream: seeded random codes (high bits set on purpose) through cpu_pack_fp6.
    gen = torch.Generator(device="cpu").manual_seed(7)
    codes = torch.randint(0, 256, (37, 128), generator=gen, dtype=torch.uint8)
    out["pack_codes"] = codes.numpy()
    out["pack_bytes"] = ref.cpu_pack_fp6(codes).numpy()
    out["pack_1234"] = ref.cpu_pack_fp6(torch.tensor([1, 2, 3, 4], dtype=torch.uint8)).numpy()

    # W6A6 decoded GEMM exactly as the reference's reference_gemm computes it.
    gen = torch.Generator(device="cpu").manual_seed(11)
    a_codes = torch.randint(0, 64, (24, 256), generator=gen, dtype=torch.uint8)
    b_codes = torch.randint(0, 64, (40, 256), generator=gen, dtype=torch.uint8)
    sfa = torch.randint(120, 135, (24, 8), generator=gen, dtype=torch.uint8)
    sfb = torch.randint(120, 135, (40, 8), generator=gen, dtype=torch.uint8)
    out["w6a6_a_codes"], out["w6a6_b_codes"] = a_codes.numpy(), b_codes.numpy()
    out["w6a6_sfa"], out["w6a6_sfb"] = sfa.numpy(), sfb.numpy()
    out["w6a6_out_f16_bits"] = (
        ref.reference_gemm(a_codes, b_codes, sfa, sfb, torch.float16).view(torch.int16).numpy()
    )

    # The CPU-runnable correctness GEMM: M=16, N=1024, K=2048, seed 0.  Codes come
    # from the oracle quantizers; the decode + FP32 matmul + BF16 cast is the
    # reference's (decode_e3m2 / decode_ue8m0 / float8 view, tests/test_ops.py:1426-1443).
    gen = torch.Generator(device="cpu").manual_seed(0)
    a = torch.randn((16, 2048), generator=gen, dtype=torch.float32).to(torch.bfloat16)
    w = (torch.randn((1024, 2048), generator=gen, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    a_q, a_s = oracle.quantize_mxfp8(a)
    w_q, w_s = oracle.quantize_mxfp6(w)
    a_deq = torch.from_numpy(a_q).view(torch.float8_e4m3fn).float() * ref.decode_ue8m0(
        torch.from_numpy(a_s)
    ).repeat_interleave(32, dim=1)
    w_deq = ref.decode_e3m2(torch.from_numpy(w_q)) * ref.decode_ue8m0(
        torch.from_numpy(w_s)
    ).repeat_interleave(32, dim=1)
    out["c1_out_bf16_bits"] = (a_deq @ w_deq.t()).to(torch.bfloat16).view(torch.int16).numpy()
    out["c1_out_f32"] = (a_deq @ w_deq.t()).numpy()
    # The reference test's own quantizer cross-check (tests/test_ops.py:1460-1467):
    # codes == (x / scale).to(float8_e4m3fn).
    scales = ref.decode_ue8m0(torch.from_numpy(a_s)).repeat_interleave(32, dim=1)
    out["c1_a_codes_by_reference_formula"] = (
        (a.float() / scales).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    )
    out["c1_a_scales"] = a_s
    out["c1_w_codes_crc"] = np.array(
        [int(np.bitwise_xor.reduce(w_q.reshape(-1).astype(np.uint32) * np.arange(1, w_q.size + 1, dtype=np.uint32)))],
        dtype=np.uint32,
    )
    np.savez_compressed(HERE / "reference_helpers.npz", **out)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <checkout of the reference project>")
    reference = Path(sys.argv[1])
    make_cvt_tables()
    make_reference_fixtures(reference)
    for name in ("cvt_tables.npz", "reference_helpers.npz"):
        print(name, (HERE / name).stat().st_size, "bytes")
