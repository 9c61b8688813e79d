"""The C++ header include/spark/kernels.h compiles and links against the library with the
reference's signatures, and turns status codes into the reference's exception types. No GPU."""

import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SRC = r'''
#include <cstdio>
#include <cstring>
#include "spark/kernels.h"
// the reference's signatures, as function-pointer types: a mismatch fails to compile
using W4 = void (*)(const __nv_bfloat16*, const int32_t*, const __nv_bfloat16*, const uint8_t*, __nv_bfloat16*, int, int, int, int, cudaStream_t);
using F8 = void (*)(const __nv_fp8_e4m3*, const __nv_fp8_e4m3*, __nv_bfloat16*, int, int, int, const float*, const float*, int, cudaStream_t);
using F8MX = void (*)(const __nv_fp8_e4m3*, const __nv_fp8_e4m3*, __nv_bfloat16*, int, int, int, const float*, const float*, const unsigned char*, const unsigned char*, int, cudaStream_t);
using F4 = void (*)(const unsigned char*, const unsigned char*, __nv_bfloat16*, int, int, int, const unsigned char*, const unsigned char*, const float*, const float*, int, int, cudaStream_t);
using F4Q = void (*)(const __nv_bfloat16*, unsigned char*, unsigned char*, int, int, const float*, int, cudaStream_t, unsigned*, float*);
using F8Q = void (*)(const __nv_bfloat16*, unsigned char*, void*, unsigned*, int, int, int, cudaStream_t);
int main() {
    W4 a = &spark::w4gemm_bf16; F8 b = &spark::fp8gemm; F8MX c = &spark::fp8gemm_mx; F4 d = &spark::fp4gemm;
    F4Q e = &spark::fp4_quantize; F8Q f = &spark::fp8_quantize;
    if (!a || !b || !c || !d || !e || !f) return 1;
    if (spark::w4gemm_num_variants() != 4 || spark::fp8gemm_num_variants() != 5 || spark::fp4gemm_num_variants() != 3) return 2;
    if (spark::kW4GroupSize != 128 || spark::fp4_scale_bytes(200, 256, spark::FP4_NVFP4) != 4096) return 3;
    if (spark::decode_need_ctas(24576, spark::DECODE_DEVICE_RTX5090) != 64) return 4;
    alignas(16) static char buf[64];
    try {  // K % 128 != 0: host validation -> std::invalid_argument, before any CUDA call
        spark::w4gemm_bf16((const __nv_bfloat16*)buf, (const int32_t*)buf, (const __nv_bfloat16*)buf, nullptr,
                           (__nv_bfloat16*)buf, 1, 16, 100, 2, nullptr);
        return 5;
    } catch (const std::invalid_argument& ex) {
        if (!std::strstr(ex.what(), "128")) return 6;
    }
    std::puts("cpp api ok");
    return 0;
}
'''


def test_cpp_header_compiles_links_and_throws(tmp_path):
    src = tmp_path / "api.cu"
    src.write_text(SRC)
    exe = tmp_path / "api"
    libdir = os.path.join(ROOT, "5090-blackwell-kernels_b200", "lib")
    cmd = ["nvcc", "-std=c++17", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe), "-L", libdir,
           "-lspark_b200", "-Xlinker", f"-rpath={libdir}"]
    subprocess.run(cmd, check=True, capture_output=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0 and "cpp api ok" in out.stdout, (out.returncode, out.stdout, out.stderr)
