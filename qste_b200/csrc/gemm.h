// Internal interface between the projection entry points and the GEMM kernels.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace qste {

// Every product is  C[i, j] = sum_k (A(i, k) * cs[k]) * sign(bits)(j, k).
enum TcKind {
  TC_FORWARD = 0,    // A = X [I, K] row-major;   bits [J, K/8]: k is the packed dimension
  TC_TRANSPOSE = 1,  // A = dY [I, K] row-major;  bits [K, J/8]: j is the packed dimension
  TC_EVIDENCE = 2    // A(i, k) = dY[k * I + i];   bits [K, J/8]: j is the packed dimension
};

struct TcProblem {
  int kind;
  const void* a;
  int a_dtype;
  const void* a_prepared;       // optional: A already re-encoded as fp16(A * a_prepared_mult[0])
  const float* a_prepared_mult; // device {2^a, 2^-a} that goes with a_prepared
  const uint8_t* bits;
  int64_t bit_pitch;
  const float* contraction_scale;  // cs[k] or NULL
  const float* out_scale;          // per output column j (forward) or NULL
  const float* out_bias;           // per output column j (forward) or NULL
  const float* row_add;            // per output row i, added before the row scale (evidence) or NULL
  const float* row_scale;          // per output row i (evidence) or NULL
  const uint8_t* inner_bits;       // [I, J/8]: also emit inner_out[i] = sum_j (acc + row_add) * sign
  float* inner_out;
  void* out;
  int out_dtype;
  int64_t I, J, K;
  char* workspace;
  unsigned long long* diagnostics;  // device counter of waits that gave up
};

size_t tc_workspace(int kind, int64_t I, int64_t J, int64_t K, int dtype);
// the same without room for a re-encoded copy of A (the caller passes a_prepared)
size_t tc_workspace_prepared(int kind, int64_t I, int64_t J, int64_t K);
// amax_slot holds the largest |A| (bits of a float, see column_sums); writes a_mult = {2^a, 2^-a}
// and out_half = fp16(A * 2^a) for a bf16 A of `count` elements
int tc_prepare_half(const void* a_bf16, int64_t count, const unsigned* amax_slot, float* a_mult,
                    void* out_half, cudaStream_t stream);
bool tc_supported(int kind, int64_t I, int64_t J, int64_t K, int dtype, const void* a,
                  const void* bits, const void* out, int out_dtype);
int tc_run(const TcProblem& problem, cudaStream_t stream);

// The largest batch of a 16-bit type the look-up-table kernel serves (2); the register-expansion
// kernel takes over above it.  QSTE_B200_LUT_TOKENS=n (0..4) moves the hand-over (for A/B timing).
int lut_max_tokens();

// Forward for 1..2 tokens (1..4 of fp32) on the CUDA cores, bound by streaming the bits (gemm_lut.cu).
bool lut_supported(int64_t samples, int64_t rows, int64_t columns, int dtype, const void* x,
                   const void* bits, const void* out, int out_dtype);
int lut_forward(const void* x, int dtype, int64_t samples, const uint8_t* packed, const float* scale,
                const float* bias, int64_t rows, int64_t columns, void* out, cudaStream_t stream);

// Forward for 3..32 tokens of a 16-bit type: warp-level MMAs with the weights expanded in registers
// (gemm_mma.cu).
bool mma_supported(int64_t samples, int64_t rows, int64_t columns, int dtype, const void* x,
                   const void* bits, const void* out, int out_dtype);
int mma_forward(const void* x, int dtype, int64_t samples, const uint8_t* packed, const float* scale,
                const float* bias, int64_t rows, int64_t columns, void* out, cudaStream_t stream);

// Coordinate evidence (with g_scale and g_bias) for 1..32 samples in one kernel on the CUDA cores,
// bound by writing the result (evidence_lut.cu; the dispatcher gives it batches up to 16).  aux = [offset (M), act_scale (M)].
bool evidence_lut_supported(int64_t samples, int64_t rows, int64_t columns, int dtype, const void* grad,
                            const float* evidence);
int evidence_lut(const void* grad, int dtype, int64_t samples, int64_t rows, const uint8_t* act_bits, const float* aux,
                 int64_t columns, const uint8_t* weight_bits, const float* weight_scale, float* evidence, float* g_scale,
                 float* g_bias, cudaStream_t stream);

// The same for 17..128 samples: warp-level MMAs with the activation signs expanded in registers
// (evidence_mma.cu).
bool evidence_mma_supported(int64_t samples, int64_t rows, int64_t columns, int dtype, const void* grad,
                            const void* act_bits, const float* evidence);
int evidence_mma(const void* grad, int dtype, int64_t samples, int64_t rows, const uint8_t* act_bits, const float* aux,
                 int64_t columns, const uint8_t* weight_bits, const float* weight_scale, float* evidence, float* g_scale,
                 float* g_bias, cudaStream_t stream);

int simt_gemm(const void* A, int a_dtype, int64_t stride_ai, int64_t stride_ak, const uint8_t* bits,
              int64_t bit_pitch, int bits_row_is_k, const float* cs, const float* os,
              const float* ob, void* C, int c_dtype, int64_t I, int64_t J, int64_t K,
              cudaStream_t stream);
bool stream_supported(int64_t samples, int64_t rows, int64_t columns, const void* packed);
bool stream_single_launch(int64_t samples, int64_t columns);
int stream_forward(const void* x, int dtype, int64_t samples, const uint8_t* packed,
                   const float* scale, const float* bias, int64_t N, int64_t K, void* out,
                   int out_dtype, cudaStream_t stream);

constexpr int kMaxSlabs = 160;
// One pass over a bf16 gradient dY [M, N] (N % 8 == 0, N <= 16384, rows 16-byte aligned):
//   out_half[m, :]  = fp16(dY[m, :] * 2^a[m]),  max |dY[m, :]| * 2^a[m] in (2^13, 2^14]
//   row_unscale[m]  = 2^-a[m]
//   row_cs[m]       = sample_scale[m] * 2^-a[m]
//   g_bias[n]       = sum_m dY[m, n]              (when g_bias is not null)
//   correction[n]   = sum_m dY[m, n] * offset[m]
// `sums` is column_sums_workspace(N) bytes of scratch; null: only the re-encoding and the two row
// vectors (row_cs[m] = 2^-a[m] when sample_scale is null).
bool prepare_rows_supported(int64_t M, int64_t N, const void* dy);
int prepare_rows(const void* dy_bf16, const float* offset, const float* sample_scale, int64_t M, int64_t N,
                 void* out_half, float* row_unscale, float* row_cs, float* g_bias, float* correction,
                 char* sums, cudaStream_t stream);

inline size_t kMaxSlabsTimesTwo() { return (size_t)kMaxSlabs * 2; }
size_t column_sums_workspace(int64_t N);
int column_sums(const void* dy, int dtype, const float* offset, int64_t M, int64_t N, float* g_bias,
                float* correction, char* workspace, unsigned* amax_slot, cudaStream_t stream);
int evidence_epilogue(float* evidence, const float* correction, const uint8_t* weight_bits,
                      const float* weight_scale, int64_t N, int64_t K, float* g_scale,
                      cudaStream_t stream);

}  // namespace qste
