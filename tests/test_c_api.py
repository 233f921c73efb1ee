"""The kernel library used from C++ without Python: a small program includes `vlrf_b200_kernels.h`, links the
library, and runs the embedding, a LayerNorm and a float32 product on memory it allocated itself."""
import shutil
import subprocess

import pytest

from vlrf_b200.csrc.build import SRC_DIR, ensure_built

pytestmark = pytest.mark.gpu

PROGRAM = r"""
#include <cmath>
#include <cstdio>
#include <vector>
#include "vlrf_b200_kernels.h"

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::printf("CUDA: %s\n", cudaGetErrorString(e_)); return 2; } } while (0)
#define OK(x) do { if ((x) != VLRF_OK) { std::printf("library: %s\n", vlrf_last_error()); return 3; } } while (0)

int main() {
    int sms = 0, major = 0, minor = 0, smem = 0;
    OK(vlrf_device_info(&sms, &major, &minor, &smem));
    const int T = 5, d = 96, V = 11, N = 7;
    std::vector<float> wte(V * d), gamma(d), beta(d), w(N * d), bias(N);
    for (int i = 0; i < V * d; ++i) wte[i] = std::sin(0.37f * i) * 2.f + 0.5f;
    for (int i = 0; i < d; ++i) { gamma[i] = 1.f + 0.01f * i; beta[i] = 0.02f * i - 0.5f; }
    for (int i = 0; i < N * d; ++i) w[i] = std::cos(0.11f * i);
    for (int i = 0; i < N; ++i) bias[i] = 0.1f * i;
    const int tokens[T] = {3, 0, 10, 3, 7};
    float *d_wte, *d_gamma, *d_beta, *d_w, *d_bias, *d_x, *d_h, *d_y;
    int *d_tok, *d_err;
    CK(cudaMalloc(&d_wte, wte.size() * 4)); CK(cudaMalloc(&d_gamma, d * 4)); CK(cudaMalloc(&d_beta, d * 4));
    CK(cudaMalloc(&d_w, w.size() * 4)); CK(cudaMalloc(&d_bias, N * 4)); CK(cudaMalloc(&d_x, T * d * 4));
    CK(cudaMalloc(&d_h, T * d * 4)); CK(cudaMalloc(&d_y, T * N * 4)); CK(cudaMalloc(&d_tok, T * 4)); CK(cudaMalloc(&d_err, 4));
    CK(cudaMemcpy(d_wte, wte.data(), wte.size() * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_gamma, gamma.data(), d * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_beta, beta.data(), d * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_w, w.data(), w.size() * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_bias, bias.data(), N * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_tok, tokens, T * 4, cudaMemcpyHostToDevice));
    CK(cudaMemset(d_err, 0, 4));
    cudaStream_t stream;
    CK(cudaStreamCreate(&stream));
    OK(vlrf_embed(d_wte, nullptr, VLRF_F32, d_tok, nullptr, d_x, T, d, V, 0, nullptr, d_err, stream));
    OK(vlrf_layernorm(d_x, nullptr, d_gamma, d_beta, d_h, VLRF_F32, T, d, 1e-5f, stream));
    OK(vlrf_gemm_simt(d_h, d_w, d_bias, nullptr, d_y, T, N, d, d, N, VLRF_F32, VLRF_F32, VLRF_ACT_NONE, stream));
    CK(cudaStreamSynchronize(stream));
    std::vector<float> y(T * N);
    int err = -1;
    CK(cudaMemcpy(y.data(), d_y, y.size() * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(&err, d_err, 4, cudaMemcpyDeviceToHost));
    double worst = 0, scale = 0;
    for (int t = 0; t < T; ++t) {
        const float* x = &wte[tokens[t] * d];
        double mean = 0, var = 0;
        for (int i = 0; i < d; ++i) mean += x[i];
        mean /= d;
        for (int i = 0; i < d; ++i) var += (x[i] - mean) * (x[i] - mean);
        const double inv = 1.0 / std::sqrt(var / d + 1e-5);
        for (int n = 0; n < N; ++n) {
            double acc = bias[n];
            for (int i = 0; i < d; ++i) acc += ((x[i] - mean) * inv * gamma[i] + beta[i]) * w[n * d + i];
            worst = std::fmax(worst, std::fabs(acc - y[t * N + n]));
            scale = std::fmax(scale, std::fabs(acc));
        }
    }
    // a size that a kernel does not take is refused with a message, and nothing runs
    const int refused = vlrf_layernorm(d_x, nullptr, d_gamma, d_beta, d_h, 7, T, d, 1e-5f, stream);
    std::printf("sms %d cc %d.%d error-word %d worst %.3e scale %.3e refused %d (%s)\n", sms, major, minor, err, worst, scale,
                refused, vlrf_last_error());
    return (err == 0 && worst <= 1e-5 * scale && refused != VLRF_OK) ? 0 : 1;
}
"""


def test_a_cpp_program_drives_the_kernels_through_the_header(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    lib = ensure_built()
    src = tmp_path / "use_kernels.cpp"
    src.write_text(PROGRAM)
    exe = tmp_path / "use_kernels"
    build = subprocess.run([nvcc, "-std=c++17", "-o", str(exe), str(src), "-I", str(SRC_DIR), str(lib),
                            "-Xlinker", f"-rpath={lib.parent}"], capture_output=True, text=True)
    assert build.returncode == 0, build.stdout + build.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "refused" in run.stdout and "unknown output dtype" in run.stdout
