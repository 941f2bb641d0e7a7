// fb_matmul_f32: bounds x constant weight.  Dispatches to the split-sign GEMM kernels.
#include "common.cuh"

#include <cstdlib>
#include <cstring>

namespace fb {
bool tc_gemm_supported(const float* a_lo, const float* a_up, const float* W, const float* c_lo, const float* c_up,
                       int64_t M, int N, int K);
int launch_split_sign_tc(const float* a_lo, const float* a_up, const float* W, const float* bias, float* c_lo,
                         float* c_up, int64_t M, int N, int K, cudaStream_t st);
int launch_split_sign_ffma(const float* a_lo, const float* a_up, const float* W, const float* bias, float* c_lo,
                           float* c_up, int64_t M, int N, int K, cudaStream_t st);

// FB_MATMUL_IMPL=ffma forces the CUDA-core kernel (exact fp32 products); default: tensor cores
// (3xTF32) for the large weight GEMM when the shape allows it.
static bool use_tensor_cores() {
  static const bool v = []() {
    const char* e = std::getenv("FB_MATMUL_IMPL");
    return !(e && std::strcmp(e, "ffma") == 0);
  }();
  return v;
}

static int split_sign_gemm(const float* a_lo, const float* a_up, const float* W, const float* bias, float* c_lo,
                           float* c_up, int64_t M, int N, int K, cudaStream_t st) {
  if (use_tensor_cores() && tc_gemm_supported(a_lo, a_up, W, c_lo, c_up, M, N, K))
    return launch_split_sign_tc(a_lo, a_up, W, bias, c_lo, c_up, M, N, K, st);
  return launch_split_sign_ffma(a_lo, a_up, W, bias, c_lo, c_up, M, N, K, st);
}
}  // namespace fb

extern "C" int fb_matmul_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                             const float* W, const float* bias, float* y_lw, float* y_uw, float* y_lb, float* y_ub,
                             int64_t rows, int Di, int Do, int Dy, void* stream) {
  if (!x_lw || !x_uw || !x_lb || !x_ub || !W || !y_lw || !y_uw || !y_lb || !y_ub) return FB_ERR_ARG;
  if (rows < 0 || Di <= 0 || Do <= 0 || Dy <= 0) return FB_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const double M = (double)rows * (Di + 1);
  fb::ProfileScope prof(fb::PK_MATMUL, 8.0 * M * Do * Dy, 4.0 * (2 * M * Do + 2 * M * Dy + (double)Do * Dy + Dy), stream);
  // weight rows: [rows * Di, Do] -> [rows * Di, Dy]; no bias on the symbolic part
  int rc = fb::split_sign_gemm(x_lw, x_uw, W, nullptr, y_lw, y_uw, rows * (int64_t)Di, Dy, Do, st);
  if (rc != FB_OK) return rc;
  // bias rows: [rows, Do] -> [rows, Dy], + bias
  return fb::split_sign_gemm(x_lb, x_ub, W, bias, y_lb, y_ub, rows, Dy, Do, st);
}
