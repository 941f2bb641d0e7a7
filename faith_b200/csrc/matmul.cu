// fb_matmul_f32: bounds x constant weight.  Dispatches to the split-sign GEMM kernels.
#include "common.cuh"

namespace fb {
int launch_split_sign_ffma(const float* a_lo, const float* a_up, const float* W, const float* bias, float* c_lo,
                           float* c_up, int64_t M, int N, int K, cudaStream_t st);
}

extern "C" int fb_matmul_f32(const float* x_lw, const float* x_uw, const float* x_lb, const float* x_ub,
                             const float* W, const float* bias, float* y_lw, float* y_uw, float* y_lb, float* y_ub,
                             int64_t rows, int Di, int Do, int Dy, void* stream) {
  if (!x_lw || !x_uw || !x_lb || !x_ub || !W || !y_lw || !y_uw || !y_lb || !y_ub) return FB_ERR_ARG;
  if (rows < 0 || Di <= 0 || Do <= 0 || Dy <= 0) return FB_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const double M = (double)rows * (Di + 1);
  fb::ProfileScope prof(fb::PK_MATMUL, 8.0 * M * Do * Dy, 4.0 * (2 * M * Do + 2 * M * Dy + (double)Do * Dy + Dy), stream);
  // weight rows: [rows * Di, Do] -> [rows * Di, Dy]; no bias on the symbolic part
  int rc = fb::launch_split_sign_ffma(x_lw, x_uw, W, nullptr, y_lw, y_uw, rows * (int64_t)Di, Dy, Do, st);
  if (rc != FB_OK) return rc;
  // bias rows: [rows, Do] -> [rows, Dy], + bias
  return fb::launch_split_sign_ffma(x_lb, x_ub, W, bias, y_lb, y_ub, rows, Dy, Do, st);
}
