"""The oracle's scalar codecs: rounding rules, saturation, and agreement with independent
implementations (torch's float8 casts and the CUDA toolkit's host-side conversion headers)."""
import math
import os
import shutil
import subprocess

import pytest
import torch

import oracle


def test_e2m1_rounds_to_nearest_even_and_saturates():
    # ties go to the code with an even mantissa: 0.25->0, 0.75->1.0, 1.25->1.0, 1.75->2.0, 2.5->2.0, 3.5->4.0, 5.0->4.0
    expect = {0.25: 0, 0.26: 1, 0.75: 2, 0.74: 1, 1.25: 2, 1.26: 3, 1.75: 4, 2.5: 4, 2.51: 5, 3.5: 6, 3.49: 5,
              5.0: 6, 5.01: 7, 6.0: 7, 100.0: 7, 0.0: 0}
    for x, code in expect.items():
        assert oracle.to_e2m1(x) == code, x
        if x:
            assert oracle.to_e2m1(-x) == (code | 8), -x
    values = [oracle.from_e2m1(c) for c in range(8)]
    assert values == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def test_e4m3_matches_torch_cast_and_saturates():
    g = torch.Generator().manual_seed(0)
    x = torch.cat([torch.rand(20000, generator=g) * 460, torch.rand(20000, generator=g) * 0.05,
                   torch.tensor([0.0, 2.0 ** -10, 2.0 ** -9, 448.0, 449.0, 1e9, 0.0009765625 * 1.5])])
    mine = torch.tensor([oracle.to_e4m3(float(v)) for v in x], dtype=torch.uint8)
    ref = x.clamp(max=448.0).to(torch.float8_e4m3fn).view(torch.uint8)
    assert torch.equal(mine, ref)
    for b in range(0x7F):
        assert oracle.to_e4m3(oracle.from_e4m3(b)) == b


def test_e8m0_rounds_up_to_power_of_two():
    assert oracle.to_e8m0(1.0) == 127
    assert oracle.to_e8m0(1.0000001) == 128
    assert oracle.to_e8m0(0.75) == 127
    assert oracle.to_e8m0(0.5) == 126
    assert oracle.to_e8m0(0.0) == 0
    assert oracle.to_e8m0(3e38) == 254
    for b in range(1, 255):
        assert oracle.to_e8m0(oracle.from_e8m0(b)) == b


def test_perm32_is_the_reference_permutation():
    # cuda_common.cuh:16-18 of the reference: (x/8)*2 + ((x%8)/2)*8 + x%2
    assert [oracle.perm32(x) for x in range(32)] == [(x // 8) * 2 + ((x % 8) // 2) * 8 + (x % 2) for x in range(32)]
    assert sorted(oracle.perm32(x) for x in range(32)) == list(range(32))


_CHECK_SRC = r"""
#include <cuda_fp8.h>
#include <cstdio>
#include <cstdint>
#include <cstring>
int main() {
    // prints: bits e4m3 e8m0 for a sweep of float bit patterns
    for (uint32_t hi = 0x30000000u; hi < 0x50000000u; hi += 0x00013579u) {
        float f; std::memcpy(&f, &hi, 4);
        unsigned a = __nv_cvt_float_to_fp8(f, __NV_SATFINITE, __NV_E4M3);
        unsigned b = __nv_cvt_float_to_e8m0(f, __NV_SATFINITE, cudaRoundPosInf);
        std::printf("%u %u %u\n", hi, a, b);
    }
    return 0;
}
"""


@pytest.mark.skipif(not os.path.exists("/usr/local/cuda/include/cuda_fp8.h") or shutil.which("g++") is None,
                    reason="CUDA toolkit headers or g++ missing")
def test_scale_codecs_match_cuda_toolkit_host_conversions(tmp_path):
    """Pins E4M3 / E8M0 encoding against the conversion routines the reference itself calls
    (__nv_fp8_e4m3(float), __nv_cvt_float_to_e8m0; nvfp4/quantization.cu:63-65, mxfp4/quantization.cu:14-16),
    using their host implementations from the CUDA toolkit headers."""
    src = tmp_path / "chk.cpp"
    src.write_text(_CHECK_SRC)
    exe = tmp_path / "chk"
    r = subprocess.run(["g++", "-O1", "-I/usr/local/cuda/include", str(src), "-o", str(exe)], capture_output=True, text=True)
    if r.returncode != 0:
        pytest.skip("toolkit headers do not compile as host-only C++ here: " + r.stderr[:200])
    lines = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split("\n")
    import struct
    n = 0
    for line in lines:
        if not line:
            continue
        bits, a, b = (int(t) for t in line.split())
        f = struct.unpack("f", struct.pack("I", bits))[0]
        assert oracle.to_e4m3(f) == a, (f, a)
        assert oracle.to_e8m0(f) == b, (f, b)
        n += 1
    assert n > 1000


def test_quantiser_layouts_and_edge_cases():
    torch.manual_seed(3)
    x = torch.randn(1, 2, 200, 128)
    x[0, 0, 3] = 0.0          # all-zero groups
    x[0, 1, 5] *= 1e4         # saturating scales
    x = x.half()
    for fmt, g in (("nvfp4", 16), ("mxfp4", 32)):
        codes, scales = oracle.quantize(x, fmt, "plain")
        assert codes.shape == (1, 2, 200, 64) and scales.shape == (1, 2, 200, 128 // g)
        assert int(codes[0, 0, 3].max()) == 0 and int(scales.view(torch.uint8)[0, 0, 3].max()) == 0
        if fmt == "nvfp4":
            assert int(scales.view(torch.uint8)[0, 1, 5].max()) == 0x7E  # 448, saturated
        # dequantised values stay within half a step of the input where nothing saturates
        cp, sp = oracle.quantize(x, fmt, "permuted")
        for p in range(64):
            logical = (p // 32) * 32 + oracle.perm32(p % 32)
            assert torch.equal(cp[0, 0, p], codes[0, 0, logical])
        # rows whose logical source lies beyond the sequence are zero
        for p in range(192, 200):
            logical = (p // 32) * 32 + oracle.perm32(p % 32)
            if logical >= 200:
                assert int(cp[0, 0, p].max()) == 0 and int(sp.view(torch.uint8)[0, 0, p].max()) == 0
        ct, st = oracle.quantize(x, fmt, "transposed")
        assert ct.shape == (1, 2, 128, 256 // 2) and st.shape == (1, 2, 128, 256 // g)
        assert int(ct[..., 100:].max()) == 0  # tokens >= 200 read as zero
        # dequantise the transposed result and compare with the input
        vals = torch.tensor([oracle.from_e2m1(c) for c in range(16)])
        lo, hi = vals[(ct & 15).long()], vals[(ct >> 4).long()]
        deq = torch.stack([lo, hi], -1).reshape(1, 2, 128, 256)
        sc = st.view(torch.uint8).long()
        scf = torch.tensor([oracle.from_e8m0(b) if fmt == "mxfp4" else (oracle.from_e4m3(b) if b != 0x7F else 0.0)
                            for b in range(256)])[sc]
        deq = deq * scf.repeat_interleave(g, dim=-1)
        err = (deq[..., :200] - x.float().transpose(2, 3)).abs()
        ok = err[0, 0] <= 0.26 * x.float().abs().max()  # coarse sanity bound: e2m1 step is at most amax/3 per group
        assert bool(ok.all())
