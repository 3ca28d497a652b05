// extern "C" entry points of the three packed-sign products and of the fused
// evidence side of the Linear backward.  Chooses between the tcgen05 kernel
// (gemm_tc.cu), the CUDA-core kernel and the small-batch streaming kernel
// (gemm_simt.cu).
#include <stdlib.h>

#include "common.cuh"
#include "gemm.h"

using namespace qste;

namespace {

constexpr size_t kHeader = 256;  // workspace[0..8): device wait-timeout counter

inline bool valid_dtype(int dtype) { return dtype_size(dtype) != 0; }

// QSTE_B200_SMALL_BATCH=0 keeps batches of 1-32 on the kernels that served them before the
// look-up-table and register-expansion kernels existed (for A/B timing).
inline bool small_batch_auto() {
  static const bool enabled = !(getenv("QSTE_B200_SMALL_BATCH") && atoi(getenv("QSTE_B200_SMALL_BATCH")) == 0);
  return enabled;
}

// The largest batch whose evidence goes to the look-up-table kernel (exact in fp32, write-bound up to
// here); above it the MMA kernel is faster.  QSTE_B200_EVIDENCE_TABLES=n (0..32) moves the hand-over.
inline int evidence_table_samples() {
  static const int samples = [] {
    const char* text = getenv("QSTE_B200_EVIDENCE_TABLES");
    const int value = text ? atoi(text) : 16;
    return value < 0 ? 0 : (value > 32 ? 32 : value);
  }();
  return samples;
}

}  // namespace

extern "C" {

size_t qste_b200_packed_linear_affine_workspace(int64_t samples, int64_t rows, int64_t columns,
                                                int dtype, int path) {
  if (path == QSTE_PATH_SIMT || path == QSTE_PATH_STREAM) return kHeader;
  return kHeader + tc_workspace(TC_FORWARD, samples, rows, columns, dtype);
}

int qste_b200_packed_linear_affine(const void* inputs, int dtype, int64_t samples,
                                   const uint8_t* packed, const float* scale, const float* bias,
                                   int64_t rows, int64_t columns, void* out, int out_dtype,
                                   int path, void* workspace, size_t workspace_bytes,
                                   qste_stream_t stream) {
  if (samples < 0 || rows < 0 || columns < 0) return QSTE_ERR_SHAPE;
  if (!valid_dtype(dtype) || !valid_dtype(out_dtype)) return QSTE_ERR_DTYPE;
  if (samples == 0 || rows == 0) return QSTE_OK;
  if (!out || !scale || (columns > 0 && (!inputs || !packed))) return QSTE_ERR_NULL;
  cudaStream_t s = as_stream(stream);
  const int64_t pitch = (columns + 7) / 8;

  // 1..2 tokens (1..4 of fp32): the look-up-table kernel (gemm_lut.cu: bits streamed once, a thread per weight row,
  // the contraction cut over a thread-block cluster); shapes it does not take fall to the older
  // streaming kernel below, larger batches to the tensor-core tiles
  if ((path == QSTE_PATH_STREAM || (path == QSTE_PATH_AUTO && small_batch_auto())) &&
      lut_supported(samples, rows, columns, dtype, inputs, packed, out, out_dtype)) {
    note_forward_kernel("lut");
    return lut_forward(inputs, dtype, samples, packed, scale, bias, rows, columns, out, s);
  }
  // 3..32 tokens of a 16-bit type: weights expanded in registers, warp-level MMAs (gemm_mma.cu)
  if ((path == QSTE_PATH_STREAM || (path == QSTE_PATH_AUTO && small_batch_auto())) &&
      mma_supported(samples, rows, columns, dtype, inputs, packed, out, out_dtype)) {
    note_forward_kernel("mma");
    return mma_forward(inputs, dtype, samples, packed, scale, bias, rows, columns, out, s);
  }
  if (path == QSTE_PATH_STREAM ||
      (path == QSTE_PATH_AUTO && stream_single_launch(samples, columns) &&
       stream_supported(samples, rows, columns, packed))) {
    if (!stream_supported(samples, rows, columns, packed)) return QSTE_ERR_UNSUPPORTED;
    note_forward_kernel("stream");
    return stream_forward(inputs, dtype, samples, packed, scale, bias, rows, columns, out, out_dtype, s);
  }
  if (path == QSTE_PATH_TENSOR || path == QSTE_PATH_AUTO) {
    const bool fits = tc_supported(TC_FORWARD, samples, rows, columns, dtype, inputs, packed, out, out_dtype);
    if (fits) {
      const size_t need = kHeader + tc_workspace(TC_FORWARD, samples, rows, columns, dtype);
      if (!workspace || workspace_bytes < need) return QSTE_ERR_WORKSPACE;
      if (!aligned(workspace, 256)) return QSTE_ERR_ALIGNMENT;
      TcProblem p = {};
      p.kind = TC_FORWARD;
      p.a = inputs; p.a_dtype = dtype; p.bits = packed; p.bit_pitch = pitch;
      p.out_scale = scale; p.out_bias = bias; p.out = out; p.out_dtype = out_dtype;
      p.I = samples; p.J = rows; p.K = columns;
      p.workspace = static_cast<char*>(workspace) + kHeader;
      p.diagnostics = static_cast<unsigned long long*>(workspace);
      note_forward_kernel("tensor");
      return tc_run(p, s);
    }
    if (path == QSTE_PATH_TENSOR) return QSTE_ERR_UNSUPPORTED;
  }
  note_forward_kernel("simt");
  return simt_gemm(inputs, dtype, columns, 1, packed, pitch, 0, nullptr, scale, bias, out, out_dtype,
                   samples, rows, columns, s);
}

size_t qste_b200_packed_transpose_workspace(int64_t samples, int64_t rows, int64_t columns,
                                            int dtype, int path) {
  if (path == QSTE_PATH_SIMT) return kHeader;
  return kHeader + tc_workspace(TC_TRANSPOSE, samples, columns, rows, dtype);
}

int qste_b200_packed_transpose(const void* inputs, int dtype, int64_t samples,
                               const uint8_t* packed, const float* row_scale, int64_t rows,
                               int64_t columns, void* out, int out_dtype, int path,
                               void* workspace, size_t workspace_bytes, qste_stream_t stream) {
  if (samples < 0 || rows < 0 || columns < 0) return QSTE_ERR_SHAPE;
  if (!valid_dtype(dtype) || !valid_dtype(out_dtype)) return QSTE_ERR_DTYPE;
  if (samples == 0 || columns == 0) return QSTE_OK;
  if (!out || (rows > 0 && (!inputs || !packed))) return QSTE_ERR_NULL;
  if (path == QSTE_PATH_STREAM) return QSTE_ERR_UNSUPPORTED;
  cudaStream_t s = as_stream(stream);
  const int64_t pitch = (columns + 7) / 8;
  if (path == QSTE_PATH_TENSOR || path == QSTE_PATH_AUTO) {
    const bool fits = tc_supported(TC_TRANSPOSE, samples, columns, rows, dtype, inputs, packed, out, out_dtype);
    if (fits) {
      const size_t need = kHeader + tc_workspace(TC_TRANSPOSE, samples, columns, rows, dtype);
      if (!workspace || workspace_bytes < need) return QSTE_ERR_WORKSPACE;
      if (!aligned(workspace, 256)) return QSTE_ERR_ALIGNMENT;
      TcProblem p = {};
      p.kind = TC_TRANSPOSE;
      p.a = inputs; p.a_dtype = dtype; p.bits = packed; p.bit_pitch = pitch;
      p.contraction_scale = row_scale; p.out = out; p.out_dtype = out_dtype;
      p.I = samples; p.J = columns; p.K = rows;
      p.workspace = static_cast<char*>(workspace) + kHeader;
      p.diagnostics = static_cast<unsigned long long*>(workspace);
      return tc_run(p, s);
    }
    if (path == QSTE_PATH_TENSOR) return QSTE_ERR_UNSUPPORTED;
  }
  return simt_gemm(inputs, dtype, rows, 1, packed, pitch, 1, row_scale, nullptr, nullptr, out,
                   out_dtype, samples, columns, rows, s);
}

size_t qste_b200_evidence_from_packed_workspace(int64_t samples, int64_t rows, int64_t columns,
                                                int dtype, int path) {
  if (path == QSTE_PATH_SIMT) return kHeader;
  return kHeader + tc_workspace(TC_EVIDENCE, rows, columns, samples, dtype);
}

int qste_b200_evidence_from_packed(const void* grad, int dtype, int64_t samples, int64_t rows,
                                   const uint8_t* packed, const float* sample_scale,
                                   int64_t columns, float* evidence, int path, void* workspace,
                                   size_t workspace_bytes, qste_stream_t stream) {
  if (samples < 0 || rows < 0 || columns < 0) return QSTE_ERR_SHAPE;
  if (!valid_dtype(dtype)) return QSTE_ERR_DTYPE;
  if (rows == 0 || columns == 0) return QSTE_OK;
  if (!evidence || (samples > 0 && (!grad || !packed))) return QSTE_ERR_NULL;
  if (path == QSTE_PATH_STREAM) return QSTE_ERR_UNSUPPORTED;
  cudaStream_t s = as_stream(stream);
  const int64_t pitch = (columns + 7) / 8;
  if (path == QSTE_PATH_TENSOR || path == QSTE_PATH_AUTO) {
    const bool fits = tc_supported(TC_EVIDENCE, rows, columns, samples, dtype, grad, packed, evidence, QSTE_F32);
    if (fits) {
      const size_t need = kHeader + tc_workspace(TC_EVIDENCE, rows, columns, samples, dtype);
      if (!workspace || workspace_bytes < need) return QSTE_ERR_WORKSPACE;
      if (!aligned(workspace, 256)) return QSTE_ERR_ALIGNMENT;
      TcProblem p = {};
      p.kind = TC_EVIDENCE;
      p.a = grad; p.a_dtype = dtype; p.bits = packed; p.bit_pitch = pitch;
      p.contraction_scale = sample_scale; p.out = evidence; p.out_dtype = QSTE_F32;
      p.I = rows; p.J = columns; p.K = samples;
      p.workspace = static_cast<char*>(workspace) + kHeader;
      p.diagnostics = static_cast<unsigned long long*>(workspace);
      return tc_run(p, s);
    }
    if (path == QSTE_PATH_TENSOR) return QSTE_ERR_UNSUPPORTED;
  }
  // A = dY^T: element (i = weight row, k = sample) lives at dY[k * rows + i]
  return simt_gemm(grad, dtype, 1, rows, packed, pitch, 1, sample_scale, nullptr, nullptr, evidence,
                   QSTE_F32, rows, columns, samples, s);
}

size_t qste_b200_linear_backward_evidence_workspace(int64_t samples, int64_t rows,
                                                    int64_t columns, int dtype, int path) {
  size_t bytes = kHeader + column_sums_workspace(rows);
  if (path != QSTE_PATH_SIMT) bytes += tc_workspace(TC_EVIDENCE, rows, columns, samples, dtype);
  return bytes;
}

int qste_b200_linear_backward_evidence(const void* grad, int dtype, int64_t samples, int64_t rows,
                                       const uint8_t* act_bits, const float* aux, int64_t columns,
                                       const uint8_t* weight_bits, const float* weight_scale,
                                       float* evidence, float* g_scale, float* g_bias, int path,
                                       void* workspace, size_t workspace_bytes,
                                       qste_stream_t stream) {
  if (samples < 0 || rows < 0 || columns < 0) return QSTE_ERR_SHAPE;
  if (!valid_dtype(dtype)) return QSTE_ERR_DTYPE;
  if (rows == 0) return QSTE_OK;
  if (!evidence && columns > 0) return QSTE_ERR_NULL;
  if (!weight_scale || (columns > 0 && !weight_bits)) return QSTE_ERR_NULL;
  if (samples > 0 && (!grad || !aux || (columns > 0 && !act_bits))) return QSTE_ERR_NULL;
  // Small batches, one launch each: up to 16 samples on the CUDA cores by look-up tables, exact in fp32
  // (evidence_lut.cu); 17..128 by warp-level MMAs (evidence_mma.cu)
  if ((path == QSTE_PATH_STREAM || (path == QSTE_PATH_AUTO && small_batch_auto())) && samples > 0 && columns > 0) {
    if (samples <= evidence_table_samples() && evidence_lut_supported(samples, rows, columns, dtype, grad, evidence))
      return evidence_lut(grad, dtype, samples, rows, act_bits, aux, columns, weight_bits, weight_scale, evidence,
                          g_scale, g_bias, as_stream(stream));
    if (evidence_mma_supported(samples, rows, columns, dtype, grad, act_bits, evidence))
      return evidence_mma(grad, dtype, samples, rows, act_bits, aux, columns, weight_bits, weight_scale, evidence,
                          g_scale, g_bias, as_stream(stream));
  }
  if (path == QSTE_PATH_STREAM) return QSTE_ERR_UNSUPPORTED;
  const size_t need = qste_b200_linear_backward_evidence_workspace(samples, rows, columns, dtype, path);
  if (!workspace || workspace_bytes < need) return QSTE_ERR_WORKSPACE;
  if (!aligned(workspace, 256)) return QSTE_ERR_ALIGNMENT;
  cudaStream_t s = as_stream(stream);
  char* base = static_cast<char*>(workspace) + kHeader;
  const size_t sums_bytes = column_sums_workspace(rows);
  float* correction = reinterpret_cast<float*>(base + (size_t)kMaxSlabsTimesTwo() * rows * sizeof(float));
  const float* offset = aux;
  const float* act_scale = aux ? aux + samples : nullptr;

  int status = column_sums(grad, dtype, offset, samples, rows, g_bias, correction, base, nullptr, s);
  if (status != QSTE_OK) return status;
  if (columns == 0) return QSTE_OK;

  const int64_t pitch = (columns + 7) / 8;
  bool done = false;
  if (path == QSTE_PATH_TENSOR || path == QSTE_PATH_AUTO) {
    if (tc_supported(TC_EVIDENCE, rows, columns, samples, dtype, grad, act_bits, evidence, QSTE_F32)) {
      TcProblem p = {};
      p.kind = TC_EVIDENCE;
      p.a = grad; p.a_dtype = dtype; p.bits = act_bits; p.bit_pitch = pitch;
      p.contraction_scale = act_scale; p.out = evidence; p.out_dtype = QSTE_F32;
      p.I = rows; p.J = columns; p.K = samples;
      p.row_add = correction; p.row_scale = weight_scale; p.inner_bits = weight_bits;
      p.inner_out = g_scale;
      p.workspace = base + sums_bytes;
      p.diagnostics = static_cast<unsigned long long*>(workspace);
      status = tc_run(p, s);
      if (status != QSTE_OK) return status;
      done = true;
    } else if (path == QSTE_PATH_TENSOR) {
      return QSTE_ERR_UNSUPPORTED;
    }
  }
  if (!done) {
    status = simt_gemm(grad, dtype, 1, rows, act_bits, pitch, 1, act_scale, nullptr, nullptr, evidence,
                       QSTE_F32, rows, columns, samples, s);
    if (status != QSTE_OK) return status;
    status = evidence_epilogue(evidence, correction, weight_bits, weight_scale, rows, columns, g_scale, s);
  }
  return status;
}

// ---- the whole backward of a converted Linear --------------------------------------------

namespace {
struct BackwardLayout { size_t sums, slots, row_vectors, half_copy, tc, total; };
BackwardLayout backward_layout(int64_t samples, int64_t rows, int64_t columns, int dtype) {
  BackwardLayout l;
  size_t at = kHeader;
  l.sums = at; at += column_sums_workspace(rows);
  l.slots = at; at += 256;
  l.row_vectors = at; at = align_up(at + (size_t)2 * samples * sizeof(float), 256);  // 2^-a[m] and sample scale * 2^-a[m]
  l.half_copy = at;
  if (dtype == QSTE_BF16) at = align_up(at + (size_t)samples * rows * 2, 256);
  l.tc = at;
  size_t a = tc_workspace_prepared(TC_TRANSPOSE, samples, columns, rows);
  size_t b = tc_workspace_prepared(TC_EVIDENCE, rows, columns, samples);
  at += a > b ? a : b;
  l.total = at;
  return l;
}
}  // namespace

size_t qste_b200_linear_backward_workspace(int64_t samples, int64_t rows, int64_t columns, int dtype) {
  if (samples <= 0 || rows <= 0 || columns <= 0) return kHeader;
  size_t fused = backward_layout(samples, rows, columns, dtype).total;
  size_t a = qste_b200_packed_transpose_workspace(samples, rows, columns, dtype, QSTE_PATH_AUTO);
  size_t b = qste_b200_linear_backward_evidence_workspace(samples, rows, columns, dtype, QSTE_PATH_AUTO);
  size_t separate = a > b ? a : b;
  return fused > separate ? fused : separate;
}

int qste_b200_linear_backward(const void* grad, int dtype, int64_t samples, int64_t rows,
                              const uint8_t* weight_bits, const float* weight_scale, int64_t columns,
                              const uint8_t* act_bits, const float* aux, void* grad_input,
                              int grad_input_dtype, float* evidence, float* g_scale, float* g_bias,
                              void* workspace, size_t workspace_bytes, qste_stream_t stream) {
  return qste_b200_linear_backward_staged(grad, dtype, samples, rows, weight_bits, weight_scale, columns, act_bits,
                                          aux, grad_input, grad_input_dtype, evidence, g_scale, g_bias, nullptr,
                                          workspace, workspace_bytes, stream);
}

// Marks "evidence, g_scale and g_bias are complete" on the stream for a caller that passed an event.
static int mark_evidence_ready(void* event, cudaStream_t s) {
  if (!event) return QSTE_OK;
  const cudaError_t error = cudaEventRecord(static_cast<cudaEvent_t>(event), s);
  if (error != cudaSuccess) { set_last_cuda_error(error, "cudaEventRecord(evidence_ready)"); return QSTE_ERR_CUDA; }
  return QSTE_OK;
}

int qste_b200_linear_backward_staged(const void* grad, int dtype, int64_t samples, int64_t rows,
                                     const uint8_t* weight_bits, const float* weight_scale, int64_t columns,
                                     const uint8_t* act_bits, const float* aux, void* grad_input,
                                     int grad_input_dtype, float* evidence, float* g_scale, float* g_bias,
                                     void* evidence_ready, void* workspace, size_t workspace_bytes,
                                     qste_stream_t stream) {
  if (samples < 0 || rows < 0 || columns < 0) return QSTE_ERR_SHAPE;
  if (!grad_input) {
    // nobody reads dX (the first layer of a model): the evidence side alone
    const int status = qste_b200_linear_backward_evidence(grad, dtype, samples, rows, act_bits, aux, columns,
                                                          weight_bits, weight_scale, evidence, g_scale, g_bias,
                                                          QSTE_PATH_AUTO, workspace, workspace_bytes, stream);
    return status != QSTE_OK ? status : mark_evidence_ready(evidence_ready, as_stream(stream));
  }
  if (!valid_dtype(dtype) || !valid_dtype(grad_input_dtype)) return QSTE_ERR_DTYPE;
  if (!workspace || workspace_bytes < qste_b200_linear_backward_workspace(samples, rows, columns, dtype))
    return QSTE_ERR_WORKSPACE;
  if (!aligned(workspace, 256)) return QSTE_ERR_ALIGNMENT;
  // (a batch of up to 128 samples takes the two separate calls: its evidence has kernels of its own)
  const bool small = small_batch_auto() && samples > 0 && columns > 0 && grad && evidence &&
                     ((samples <= evidence_table_samples() && evidence_lut_supported(samples, rows, columns, dtype, grad, evidence)) ||
                      evidence_mma_supported(samples, rows, columns, dtype, grad, act_bits, evidence));
  const bool fused = !small && dtype == QSTE_BF16 && samples > 0 && rows > 0 && columns > 0 && grad && weight_bits &&
                     weight_scale && act_bits && aux && grad_input && evidence &&
                     tc_supported(TC_TRANSPOSE, samples, columns, rows, dtype, grad, weight_bits, grad_input, grad_input_dtype) &&
                     tc_supported(TC_EVIDENCE, rows, columns, samples, dtype, grad, act_bits, evidence, QSTE_F32);
  if (!fused) {
    // any other combination: the two calls, one after the other, sharing the workspace
    int status = qste_b200_linear_backward_evidence(grad, dtype, samples, rows, act_bits, aux, columns, weight_bits,
                                                    weight_scale, evidence, g_scale, g_bias, QSTE_PATH_AUTO,
                                                    workspace, workspace_bytes, stream);
    if (status != QSTE_OK) return status;
    status = mark_evidence_ready(evidence_ready, as_stream(stream));
    if (status != QSTE_OK) return status;
    return qste_b200_packed_transpose(grad, dtype, samples, weight_bits, weight_scale, rows, columns,
                                      grad_input, grad_input_dtype, QSTE_PATH_AUTO, workspace,
                                      workspace_bytes, stream);
  }
  cudaStream_t s = as_stream(stream);
  const BackwardLayout l = backward_layout(samples, rows, columns, dtype);
  char* base = static_cast<char*>(workspace);
  float* a_mult = reinterpret_cast<float*>(base + l.slots);
  unsigned* amax_slot = reinterpret_cast<unsigned*>(base + l.slots + 16);
  float* correction = reinterpret_cast<float*>(base + l.sums + (size_t)kMaxSlabsTimesTwo() * rows * sizeof(float));
  void* half_copy = base + l.half_copy;
  const int64_t pitch = (columns + 7) / 8;

  if (prepare_rows_supported(samples, rows, grad)) {
    // One pass over dY: bias gradient, offset correction, and an fp16 re-encoding with one power
    // of two per row.  The power goes back out through the row scale of the dX epilogue and rides
    // the per-sample contraction scale of the evidence product.
    float* row_unscale = reinterpret_cast<float*>(base + l.row_vectors);
    float* row_cs = row_unscale + samples;
    int status = prepare_rows(grad, aux, aux + samples, samples, rows, half_copy, row_unscale, row_cs, g_bias,
                              correction, base + l.sums, s);
    if (status != QSTE_OK) return status;
    // The evidence product goes first: whoever reduces or applies it on another stream (the
    // all-reduce across ranks, the coordinate update) can start while dX is still being formed.
    TcProblem ev = {};
    ev.kind = TC_EVIDENCE;
    ev.a = grad; ev.a_dtype = dtype; ev.a_prepared = half_copy; ev.a_prepared_mult = nullptr;
    ev.bits = act_bits; ev.bit_pitch = pitch; ev.contraction_scale = row_cs;
    ev.out = evidence; ev.out_dtype = QSTE_F32;
    ev.I = rows; ev.J = columns; ev.K = samples;
    ev.row_add = correction; ev.row_scale = weight_scale; ev.inner_bits = weight_bits; ev.inner_out = g_scale;
    ev.workspace = base + l.tc;
    ev.diagnostics = static_cast<unsigned long long*>(workspace);
    status = tc_run(ev, s);
    if (status != QSTE_OK) return status;
    status = mark_evidence_ready(evidence_ready, s);
    if (status != QSTE_OK) return status;
    TcProblem dx = {};
    dx.kind = TC_TRANSPOSE;
    dx.a = grad; dx.a_dtype = dtype; dx.a_prepared = half_copy; dx.a_prepared_mult = nullptr;
    dx.bits = weight_bits; dx.bit_pitch = pitch; dx.contraction_scale = weight_scale;
    dx.row_scale = row_unscale;
    dx.out = grad_input; dx.out_dtype = grad_input_dtype;
    dx.I = samples; dx.J = columns; dx.K = rows;
    dx.workspace = base + l.tc;
    dx.diagnostics = static_cast<unsigned long long*>(workspace);
    return tc_run(dx, s);
  }

  // one pass over dY: bias gradient, offset correction and the largest magnitude
  cudaError_t error = cudaMemsetAsync(amax_slot, 0, sizeof(unsigned), s);
  if (error != cudaSuccess) { set_last_cuda_error(error, "cudaMemsetAsync"); return QSTE_ERR_CUDA; }
  int status = column_sums(grad, dtype, aux, samples, rows, g_bias, correction, base + l.sums, amax_slot, s);
  if (status != QSTE_OK) return status;
  // one fp16 re-encoding of dY, shared by both products
  status = tc_prepare_half(grad, samples * rows, amax_slot, a_mult, half_copy, s);
  if (status != QSTE_OK) return status;

  TcProblem ev = {};
  ev.kind = TC_EVIDENCE;
  ev.a = grad; ev.a_dtype = dtype; ev.a_prepared = half_copy; ev.a_prepared_mult = a_mult;
  ev.bits = act_bits; ev.bit_pitch = pitch; ev.contraction_scale = aux + samples;
  ev.out = evidence; ev.out_dtype = QSTE_F32;
  ev.I = rows; ev.J = columns; ev.K = samples;
  ev.row_add = correction; ev.row_scale = weight_scale; ev.inner_bits = weight_bits; ev.inner_out = g_scale;
  ev.workspace = base + l.tc;
  ev.diagnostics = static_cast<unsigned long long*>(workspace);
  status = tc_run(ev, s);
  if (status != QSTE_OK) return status;
  status = mark_evidence_ready(evidence_ready, s);
  if (status != QSTE_OK) return status;

  TcProblem dx = {};
  dx.kind = TC_TRANSPOSE;
  dx.a = grad; dx.a_dtype = dtype; dx.a_prepared = half_copy; dx.a_prepared_mult = a_mult;
  dx.bits = weight_bits; dx.bit_pitch = pitch; dx.contraction_scale = weight_scale;
  dx.out = grad_input; dx.out_dtype = grad_input_dtype;
  dx.I = samples; dx.J = columns; dx.K = rows;
  dx.workspace = base + l.tc;
  dx.diagnostics = static_cast<unsigned long long*>(workspace);
  return tc_run(dx, s);
}

}  // extern "C"
