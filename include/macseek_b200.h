/* libmacseek_b200 -- C ABI of the B200 (sm_100a) implementation of MacSeek's per-token hot path.
 *
 * Every function only ENQUEUES work on the given CUDA stream (a cudaStream_t passed as void*; NULL = the default
 * stream) and returns 0, or a negative MSB_E_* code with a message available from msb_last_error().  This is the
 * convention of the reference's host layer, whose encode_* functions "only encode into the given Enc (never
 * commit/wait)" (src/kernels/quant.hpp:3, arch.hpp:4-5, attn.hpp:3-4); a reference Buffer{buf, off} becomes the
 * device pointer buf + off, an Enc becomes the stream, and die()/abort() becomes a status code.
 * All pointers are device pointers unless a parameter is documented as host memory.  There is no CPU fallback.
 */
#ifndef MACSEEK_B200_H
#define MACSEEK_B200_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

enum { MSB_OK = 0, MSB_E_ARG = -1, MSB_E_TYPE = -2, MSB_E_CUDA = -3, MSB_E_SCRATCH = -4, MSB_E_DEVICE = -5,
       MSB_E_LIMIT = -6 };

/* Weight types: ggml type ids, as ms::q::QType (src/kernels/quant_types.hpp:10-12). */
enum { MSB_F32 = 0, MSB_F16 = 1, MSB_Q8_0 = 8, MSB_Q5_K = 13, MSB_Q6_K = 14, MSB_IQ2_XXS = 16, MSB_IQ1_S = 19,
       MSB_IQ4_NL = 20, MSB_BF16 = 30 };

const char* msb_last_error(void);
/* Library build tag, e.g. "macseek_b200 sm_100a". */
const char* msb_version(void);
/* Prepares the current device (codebook tables, status word).  Optional: every entry point does it on first use. */
int msb_init(void);
/* Synchronises the current device and returns the device-side failure word: 0, or 1/2 when a kernel abandoned a
 * bounded wait on its shared-memory ring, 3 for an abandoned peer wait.  The word is cleared by the call. */
int msb_device_status(void);

/* Block geometry: ms::q::block_elems / block_bytes / row_bytes (src/kernels/quant_types.hpp:15-36). */
int msb_block_elems(int qtype);
size_t msb_block_bytes(int qtype);
size_t msb_row_bytes(int qtype, int64_t cols);

/* out[0..n) = dequantised blocks, bit-identical with the reference's CPU ref::dequant_row
 * (tests/ref/dequant.cpp:34-120; the GPU counterpart in the reference is q_deq_f16, src/kernels/quant_mm.metal:143-154).
 * n must be a whole number of blocks; out 16-byte aligned. */
int msb_dequant(int qtype, const void* blocks, int64_t n, float* out, void* stream);

/* y[rows] (+)= W[rows x cols] . x   -- ms::q::encode_matvec (src/kernels/quant.hpp:27-30, quant.mm:70-95).
 * W: raw GGUF block rows (2-byte aligned).  groups > 1: block-diagonal, row group g reads x[g*cols .. g*cols+cols).
 * Preconditions as the reference (quant.mm:73): cols a multiple of the block size, rows % groups == 0. */
int msb_matvec(int qtype, const void* W, int rows, int cols, const float* x, float* y, int accumulate, int groups,
               void* stream);
/* Y[n x rows] (+)= X[n x cols*groups] . W^T, 1 <= n <= 16 -- ms::q::encode_matvec_n (quant.hpp:32-35, quant.mm:129-156).
 * Row stride of X = cols*groups, of Y = rows. */
int msb_matvec_n(int qtype, const void* W, int rows, int cols, const float* X, float* Y, int n, int accumulate,
                 int groups, void* stream);

#ifdef __cplusplus
}
#endif
#endif
