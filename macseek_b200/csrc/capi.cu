// extern "C" surface of libmacseek_b200 (declared in include/macseek_b200.h).
#include "msb_common.cuh"
#include "../../include/macseek_b200.h"

namespace msb {
const char* last_error_text();
int dequant(int t, const void* src, int64_t n, float* out, cudaStream_t st);
int matvec_n(int t, const void* W, int rows, int cols, const float* X, int64_t x_stride, float* Y, int64_t y_stride,
             int n, int accumulate, int groups, cudaStream_t st);
}  // namespace msb

using namespace msb;

extern "C" {

const char* msb_last_error(void) { return last_error_text(); }
const char* msb_version(void) { return "macseek_b200 sm_100a"; }

int msb_init(void) {
  Tables t;
  return get_tables(&t);
}

int msb_device_status(void) {
  Tables t;
  int rc = get_tables(&t);
  if (rc) return rc;
  MSB_CUDA(cudaDeviceSynchronize());
  int v = 0;
  MSB_CUDA(cudaMemcpy(&v, t.status, sizeof v, cudaMemcpyDeviceToHost));
  if (v) MSB_CUDA(cudaMemset(t.status, 0, sizeof v));
  return v;
}

int msb_block_elems(int qtype) { return type_known(qtype) ? block_elems(qtype) : 0; }
size_t msb_block_bytes(int qtype) { return (size_t)block_bytes(qtype); }
size_t msb_row_bytes(int qtype, int64_t cols) { return type_known(qtype) ? row_bytes(qtype, cols) : 0; }

int msb_dequant(int qtype, const void* blocks, int64_t n, float* out, void* stream) {
  return dequant(qtype, blocks, n, out, (cudaStream_t)stream);
}

int msb_matvec(int qtype, const void* W, int rows, int cols, const float* x, float* y, int accumulate, int groups,
               void* stream) {
  return matvec_n(qtype, W, rows, cols, x, (int64_t)cols * groups, y, rows, 1, accumulate, groups, (cudaStream_t)stream);
}

int msb_matvec_n(int qtype, const void* W, int rows, int cols, const float* X, float* Y, int n, int accumulate,
                 int groups, void* stream) {
  if (n < 1 || n > 16) return fail(kErrArg, "matvec_n: n = %d outside 1..16", n);
  return matvec_n(qtype, W, rows, cols, X, (int64_t)cols * groups, Y, rows, n, accumulate, groups, (cudaStream_t)stream);
}

}  // extern "C"
