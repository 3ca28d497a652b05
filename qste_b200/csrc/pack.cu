// Bit packing and the small row-local kernels of the binary-layer path.
//
// This translation unit is compiled with -fmad=false: the bits written by
// pack_affine_rows depend on the exact fp32 value of each row mean, so every
// sum below is formed in the same order, with the same roundings, as the
// reference's CPU kernel (src/qste/kernels/cpu.cpp:143-203) and nothing may be
// contracted into an FMA.
#include <type_traits>

#include "common.cuh"

namespace qste {

// ---------------------------------------------------------------------------
// pack_coordinate / pack_bits: one thread per output byte
// ---------------------------------------------------------------------------

template <bool kSigned>
__global__ void pack_bytes_kernel(const uint8_t* __restrict__ source, int64_t rows, int64_t columns,
                                  uint8_t* __restrict__ packed) {
  const int64_t stride = (columns + 7) >> 3;
  const int64_t total = rows * stride;
  const bool fast = (columns & 7) == 0 && (reinterpret_cast<uintptr_t>(source) & 7) == 0;
  for (int64_t q = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; q < total;
       q += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = q / stride, byte = q - row * stride;
    const int64_t column0 = byte * 8;
    unsigned bits = 0;
    if (fast) {
      const uint2 raw = *reinterpret_cast<const uint2*>(source + row * columns + column0);
      const unsigned words[2] = {raw.x, raw.y};
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        const unsigned value = (words[b >> 2] >> (8 * (b & 3))) & 0xffu;
        const unsigned set = kSigned ? ((value >> 7) ^ 1u) : (value != 0u);
        bits |= set << b;
      }
    } else {
      for (int b = 0; b < 8; ++b) {
        const int64_t column = column0 + b;
        if (column < columns) {
          const unsigned value = source[row * columns + column];
          const unsigned set = kSigned ? ((value >> 7) ^ 1u) : (value != 0u);
          bits |= set << b;
        }
      }
    }
    packed[q] = (uint8_t)bits;
  }
}

// The same for matrices whose every row is a multiple of 64 bytes and 16-byte aligned (all the
// layer widths in practice): a thread turns 64 source bytes into 8 packed ones.  Its four
// 16-byte loads are issued before any of them is used, so four times the bytes are in flight
// per thread (the byte-per-thread kernel reached 22 % of DRAM bandwidth at 14336 x 4096: one
// 8-byte load per thread is too little to cover the latency), and the 8-byte store fills a
// sector with four threads instead of thirty-two.
template <bool kSigned>
__global__ void __launch_bounds__(256)
pack_bytes_wide_kernel(const uint4* __restrict__ source, int64_t groups, uint2* __restrict__ packed) {
  for (int64_t g = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; g < groups; g += (int64_t)gridDim.x * blockDim.x) {
    uint4 raw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) raw[i] = source[4 * g + i];
    unsigned out[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const unsigned words[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
      unsigned bits = 0;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        // the top bit of each byte (sign) or "byte != 0", gathered into four consecutive bits
        unsigned flags;
        if (kSigned) flags = (~words[w] >> 7) & 0x01010101u;
        else flags = (((words[w] & 0x7f7f7f7fu) + 0x7f7f7f7fu) | words[w]) >> 7 & 0x01010101u;
        bits |= ((flags * 0x10204080u) >> 28) << (4 * w);
      }
      out[i >> 1] |= bits << (16 * (i & 1));
    }
    packed[g] = make_uint2(out[0], out[1]);
  }
}

// ---------------------------------------------------------------------------
// pack_affine_rows
// ---------------------------------------------------------------------------
//
// A warp owns 8 rows.  Lane (r, j) = (lane / 4, lane % 4) walks the strided sum
// s_j of row r exactly as cpu.cpp:165-172 does (s_j += x[4i + j] for ascending
// i, the ragged tail into s_0), so mean = ((s0 + s1) + s2) + s3) * (1 / columns)
// is bit-identical.  The second pass builds each byte and the two absolute
// deviation sums d0 / d1 in the order of cpu.cpp:177-199.  Rows are streamed
// through a per-warp shared-memory tile of 8 x 256 floats so that global loads
// stay coalesced; the tile pitch (260 floats) makes both access patterns
// conflict-free.

constexpr int kTileColumns = 256;
constexpr int kTilePitch = 260;
constexpr int kRowsPerWarp = 8;
constexpr int kPackWarps = 4;

template <typename T>
__device__ __forceinline__ void load_row_tile(const T* __restrict__ x, int64_t row0, int64_t rows,
                                              int64_t columns, int64_t c0,
                                              float (*tile)[kTilePitch], int lane, bool vector_ok) {
  constexpr int kVec = 16 / sizeof(T);
  constexpr int kChunks = kTileColumns / kVec / 32;
#pragma unroll
  for (int rr = 0; rr < kRowsPerWarp; ++rr) {
    const int64_t row = row0 + rr;
#pragma unroll
    for (int q = 0; q < kChunks; ++q) {
      const int local = (q * 32 + lane) * kVec;
      const int64_t c = c0 + local;
      float v[kVec];
#pragma unroll
      for (int e = 0; e < kVec; ++e) v[e] = 0.0f;
      if (row < rows && c < columns) {
        const T* p = x + row * columns + c;
        if (vector_ok && c + kVec <= columns) {
          const uint4 raw = *reinterpret_cast<const uint4*>(p);
          const T* lanes = reinterpret_cast<const T*>(&raw);
#pragma unroll
          for (int e = 0; e < kVec; ++e) v[e] = DType<T>::load(lanes + e);
        } else {
          for (int e = 0; e < kVec; ++e)
            if (c + e < columns) v[e] = DType<T>::load(p + e);
        }
      }
      float4* destination = reinterpret_cast<float4*>(&tile[rr][local]);
#pragma unroll
      for (int e = 0; e < kVec / 4; ++e)
        destination[e] = make_float4(v[4 * e], v[4 * e + 1], v[4 * e + 2], v[4 * e + 3]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kPackWarps * 32)
pack_affine_rows_kernel(const T* __restrict__ x, int64_t rows, int64_t columns,
                        uint8_t* __restrict__ packed, float* __restrict__ offset,
                        float* __restrict__ scale, int vector_ok) {
  __shared__ __align__(16) float tiles[kPackWarps][kRowsPerWarp][kTilePitch];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row0 = ((int64_t)blockIdx.x * kPackWarps + warp) * kRowsPerWarp;
  if (row0 >= rows) return;
  float (*tile)[kTilePitch] = tiles[warp];
  const int r = lane >> 2, j = lane & 3;
  const int64_t my_row = row0 + r;
  const bool valid = my_row < rows;
  const int64_t stride = (columns + 7) >> 3;
  const int64_t main4 = columns & ~(int64_t)3;
  const float inverse = 1.0f / (float)(columns > 1 ? columns : 1);

  // pass 1: the four strided sums
  float s = 0.0f;
  for (int64_t c0 = 0; c0 < columns; c0 += kTileColumns) {
    load_row_tile<T>(x, row0, rows, columns, c0, tile, lane, vector_ok != 0);
    __syncwarp();
    const int64_t remaining = columns - c0;
    const int width = remaining < kTileColumns ? (int)remaining : kTileColumns;
    const int64_t main_left = main4 - c0;
    const int limit = main_left <= 0 ? 0 : (main_left < kTileColumns ? (int)main_left : kTileColumns);
    const float* line = tile[r];
#pragma unroll 8
    for (int c = j; c < limit; c += 4) s += line[c];
    if (j == 0)
      for (int c = limit; c < width; ++c) s += line[c];
    __syncwarp();
  }
  const int base = lane & ~3;
  const float s0 = __shfl_sync(0xffffffffu, s, base);
  const float s1 = __shfl_sync(0xffffffffu, s, base + 1);
  const float s2 = __shfl_sync(0xffffffffu, s, base + 2);
  const float s3 = __shfl_sync(0xffffffffu, s, base + 3);
  const float mean = (s0 + s1 + s2 + s3) * inverse;

  // pass 2: bits and the two deviation sums
  const int64_t full = columns >> 3;
  const bool word_stores = (stride & 3) == 0 && (reinterpret_cast<uintptr_t>(packed) & 3) == 0;
  float d = 0.0f;
  unsigned tail_bits = 0;
  for (int64_t c0 = 0; c0 < columns; c0 += kTileColumns) {
    load_row_tile<T>(x, row0, rows, columns, c0, tile, lane, vector_ok != 0);
    __syncwarp();
    const int64_t byte0 = c0 >> 3;
    const int64_t bytes_left = full - byte0;
    const int nbytes = bytes_left <= 0 ? 0 : (bytes_left < 32 ? (int)bytes_left : 32);
    const float* line = tile[r];
    unsigned word = 0;
    for (int b = 0; b < nbytes; ++b) {
      unsigned nibble = 0;
      if (j < 2) {
        const float4 v = *reinterpret_cast<const float4*>(line + 8 * b + 4 * j);
        const float e0 = v.x - mean, e1 = v.y - mean, e2 = v.z - mean, e3 = v.w - mean;
        d += fabsf(e0) + fabsf(e1) + fabsf(e2) + fabsf(e3);
        nibble = (e0 >= 0.0f ? 1u : 0u) | (e1 >= 0.0f ? 2u : 0u) | (e2 >= 0.0f ? 4u : 0u) |
                 (e3 >= 0.0f ? 8u : 0u);
      }
      const unsigned low = __shfl_sync(0xffffffffu, nibble, base);
      const unsigned high = __shfl_sync(0xffffffffu, nibble, base + 1);
      const unsigned byte = low | (high << 4);
      if (word_stores) {
        word |= byte << (8 * (b & 3));
        if ((b & 3) == 3) {
          if (j == 0 && valid)
            *reinterpret_cast<uint32_t*>(packed + my_row * stride + byte0 + (b & ~3)) = word;
          word = 0;
        }
      } else if (j == 0 && valid) {
        packed[my_row * stride + byte0 + b] = (uint8_t)byte;
      }
    }
    if (word_stores && (nbytes & 3) != 0 && j == 0 && valid) {
      // ragged end of the full bytes inside a word: store byte by byte
      const int first = nbytes & ~3;
      for (int b = first; b < nbytes; ++b)
        packed[my_row * stride + byte0 + b] = (uint8_t)((word >> (8 * (b & 3))) & 0xffu);
    }
    // the ragged tail of the row (columns % 8 elements) lives in the last tile
    if (j == 0 && full * 8 >= c0 && full * 8 < c0 + kTileColumns && full < stride) {
      const int start = (int)(full * 8 - c0);
      const int width = (int)((columns - c0) < kTileColumns ? (columns - c0) : kTileColumns);
      for (int c = start; c < width; ++c) {
        const float centered = line[c] - mean;
        d += fabsf(centered);
        if (centered >= 0.0f) tail_bits |= 1u << (c - start);
      }
      if (valid) packed[my_row * stride + full] = (uint8_t)tail_bits;
    }
    __syncwarp();
  }
  const float d0 = __shfl_sync(0xffffffffu, d, base);
  const float d1 = __shfl_sync(0xffffffffu, d, base + 1);
  if (j == 0 && valid) {
    offset[my_row] = mean;
    scale[my_row] = (d0 + d1) * inverse;
  }
}

// ---------------------------------------------------------------------------
// pack_affine_rows, rows that start on 16-byte boundaries
// ---------------------------------------------------------------------------
//
// Same chains, same order, same roundings as the kernel above; only the data movement
// differs.  The rows are streamed through a per-warp ring of four stages filled with 16-byte
// cp.async in the input's own dtype (256 bytes of each of the warp's 8 rows per stage), so
// the loads of the next three stages are in flight while a stage is consumed, and the values
// are converted to fp32 when they are read.  Rows are 16 bytes further apart than their
// length, which spreads the 8 rows of a warp over all banks.  The ring is small (8.5 KB per
// warp) because the kernel is bound by instruction latency, not bandwidth: what it needs is
// many warps per SM.

constexpr int kAsyncStages = 4;
constexpr int kAsyncWarps = 2;
constexpr int kAsyncRowBytes = 256;
constexpr int kAsyncPitch = kAsyncRowBytes + 16;

__device__ __forceinline__ void pack_cp_async16(void* smem, const void* global) {
  const unsigned address = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(address), "l"(global) : "memory");
}
__device__ __forceinline__ void pack_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void pack_cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// four consecutive elements starting at a 4-element boundary of a shared-memory row, as fp32
template <typename T>
__device__ __forceinline__ float4 load_quad(const uint8_t* line, int element) {
  if constexpr (sizeof(T) == 4) {
    return *reinterpret_cast<const float4*>(line + element * 4);
  } else {
    const uint2 raw = *reinterpret_cast<const uint2*>(line + element * 2);
    float4 v;
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      v.x = __uint_as_float(raw.x << 16); v.y = __uint_as_float(raw.x & 0xffff0000u);
      v.z = __uint_as_float(raw.y << 16); v.w = __uint_as_float(raw.y & 0xffff0000u);
    } else {
      v.x = __half2float(__ushort_as_half((unsigned short)(raw.x & 0xffffu)));
      v.y = __half2float(__ushort_as_half((unsigned short)(raw.x >> 16)));
      v.z = __half2float(__ushort_as_half((unsigned short)(raw.y & 0xffffu)));
      v.w = __half2float(__ushort_as_half((unsigned short)(raw.y >> 16)));
    }
    return v;
  }
}

template <typename T>
__global__ void __launch_bounds__(kAsyncWarps * 32)
pack_affine_rows_async_kernel(const T* __restrict__ x, int64_t rows, int64_t columns,
                              uint8_t* __restrict__ packed, float* __restrict__ offset,
                              float* __restrict__ scale) {
  constexpr int kVec = 16 / (int)sizeof(T);                  // elements per 16-byte chunk
  constexpr int kTileCols = kAsyncRowBytes / (int)sizeof(T); // columns per stage
  __shared__ __align__(16) uint8_t rings[kAsyncWarps][kAsyncStages][kRowsPerWarp][kAsyncPitch];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row0 = ((int64_t)blockIdx.x * kAsyncWarps + warp) * kRowsPerWarp;
  if (row0 >= rows) return;
  uint8_t (*ring)[kRowsPerWarp][kAsyncPitch] = rings[warp];
  const int r = lane >> 2, j = lane & 3;
  const int64_t my_row = row0 + r;
  const bool valid = my_row < rows;
  const int64_t stride = (columns + 7) >> 3;
  const int64_t tiles = (columns + kTileCols - 1) / kTileCols;
  const float inverse = 1.0f / (float)(columns > 1 ? columns : 1);

  // a stage holds 16 chunks of each of the 8 rows: lane l fetches chunk l % 16 of rows l / 16,
  // l / 16 + 2, ...; chunks past the row's end become zeros
  auto issue = [&](int64_t t) {
    const int slot = (int)(t % kAsyncStages);
    const int chunk = lane & 15;
    const int64_t c = t * kTileCols + (int64_t)chunk * kVec;
#pragma unroll
    for (int pair = 0; pair < kRowsPerWarp / 2; ++pair) {
      const int rr = 2 * pair + (lane >> 4);
      uint8_t* destination = &ring[slot][rr][chunk * 16];
      if (row0 + rr < rows && c < columns)
        pack_cp_async16(destination, x + (row0 + rr) * columns + c);
      else
        *reinterpret_cast<uint4*>(destination) = make_uint4(0u, 0u, 0u, 0u);
    }
    pack_cp_async_commit();
  };
  // always kAsyncStages - 1 groups in the prologue and one per iteration (empty past the end),
  // so that "at most kAsyncStages - 1 groups pending" means "tile t has landed"
  auto walk = [&](auto body) {
    for (int64_t t = 0; t < kAsyncStages - 1; ++t) {
      if (t < tiles) issue(t); else pack_cp_async_commit();
    }
    for (int64_t t = 0; t < tiles; ++t) {
      if (t + kAsyncStages - 1 < tiles) issue(t + kAsyncStages - 1); else pack_cp_async_commit();
      pack_cp_async_wait<kAsyncStages - 1>();
      __syncwarp();
      body(t, ring[t % kAsyncStages][r]);
      __syncwarp();
    }
    pack_cp_async_wait<0>();
    __syncwarp();
  };

  // pass 1: the four strided sums (columns is a multiple of 4 here: no ragged tail)
  float s = 0.0f;
  walk([&](int64_t, const uint8_t* line) {
    const T* elements = reinterpret_cast<const T*>(line) + j;
#pragma unroll
    for (int i = 0; i < kTileCols / 4; ++i) s += DType<T>::load(elements + 4 * i);
  });
  const int base = lane & ~3;
  const float s0 = __shfl_sync(0xffffffffu, s, base);
  const float s1 = __shfl_sync(0xffffffffu, s, base + 1);
  const float s2 = __shfl_sync(0xffffffffu, s, base + 2);
  const float s3 = __shfl_sync(0xffffffffu, s, base + 3);
  const float mean = (s0 + s1 + s2 + s3) * inverse;

  // pass 2: bits and the two deviation sums; lane j < 2 owns nibble j of every byte
  const int64_t full = columns >> 3;
  const bool word_stores = (stride & 3) == 0 && (reinterpret_cast<uintptr_t>(packed) & 3) == 0;
  float d = 0.0f;
  walk([&](int64_t t, const uint8_t* line) {
    const int64_t byte0 = t * (kTileCols / 8);
    const int64_t bytes_left = full - byte0;
    const int nbytes = bytes_left <= 0 ? 0 : (bytes_left < kTileCols / 8 ? (int)bytes_left : kTileCols / 8);
    // one nibble: its four sign bits and the sum of its four absolute deviations
    auto nibble_at = [&](int b, int nibble, float& deviation) {
      const float4 v = load_quad<T>(line, 8 * b + 4 * nibble);
      const float e0 = v.x - mean, e1 = v.y - mean, e2 = v.z - mean, e3 = v.w - mean;
      deviation = fabsf(e0) + fabsf(e1) + fabsf(e2) + fabsf(e3);
      return (e0 >= 0.0f ? 1u : 0u) | (e1 >= 0.0f ? 2u : 0u) | (e2 >= 0.0f ? 4u : 0u) | (e3 >= 0.0f ? 8u : 0u);
    };
    auto nibble_of = [&](int b) {   // lanes j < 2: nibble j of byte b, and its share of d
      float deviation;
      const unsigned bits = nibble_at(b, j, deviation);
      d += deviation;
      return bits;
    };
    // Four bytes at a time, all four lanes of the row at work: lane j takes nibble j % 2 of the
    // bytes b + j / 2 and b + j / 2 + 2.  The deviation sums stay on lanes 0 and 1, which add
    // their own two nibbles and the two handed over by lanes 2 and 3 in byte order, i.e. in the
    // order in which one lane would have added them.
    const int nibble = j & 1, odd = j >> 1;
    int b = 0;
    for (; b + 4 <= nbytes; b += 4) {
      float first, second;
      unsigned word = nibble_at(b + odd, nibble, first) << (8 * odd + 4 * nibble);
      word |= nibble_at(b + odd + 2, nibble, second) << (8 * (odd + 2) + 4 * nibble);
      const float first_odd = __shfl_sync(0xffffffffu, first, base + 2 + nibble);
      const float second_odd = __shfl_sync(0xffffffffu, second, base + 2 + nibble);
      if (j < 2) {
        d += first;
        d += first_odd;
        d += second;
        d += second_odd;
      }
      word |= __shfl_xor_sync(0xffffffffu, word, 1);
      word |= __shfl_xor_sync(0xffffffffu, word, 2);
      if (j == 0 && valid) {
        uint8_t* destination = packed + my_row * stride + byte0 + b;
        if (word_stores) {
          *reinterpret_cast<uint32_t*>(destination) = word;
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) destination[k] = (uint8_t)((word >> (8 * k)) & 0xffu);
        }
      }
    }
    if (b < nbytes) {
      unsigned word = 0;
      if (j < 2)
        for (int k = 0; b + k < nbytes; ++k) word |= nibble_of(b + k) << (8 * k + 4 * j);
      const unsigned both = word | __shfl_sync(0xffffffffu, word, base + 1);
      if (j == 0 && valid)
        for (int k = 0; b + k < nbytes; ++k)
          packed[my_row * stride + byte0 + b + k] = (uint8_t)((both >> (8 * k)) & 0xffu);
    }
    // four elements left over when columns % 8 == 4 (fp32 rows only): they live in the last tile
    if (j == 0 && full < stride && full >= byte0 && full < byte0 + kTileCols / 8) {
      const int start = (int)(full * 8 - t * kTileCols);
      const int width = (int)(columns - t * kTileCols);
      unsigned tail_bits = 0;
      for (int c = start; c < width; ++c) {
        const float centered = DType<T>::load(reinterpret_cast<const T*>(line) + c) - mean;
        d += fabsf(centered);
        if (centered >= 0.0f) tail_bits |= 1u << (c - start);
      }
      if (valid) packed[my_row * stride + full] = (uint8_t)tail_bits;
    }
  });
  const float d0 = __shfl_sync(0xffffffffu, d, base);
  const float d1 = __shfl_sync(0xffffffffu, d, base + 1);
  if (j == 0 && valid) {
    offset[my_row] = mean;
    scale[my_row] = (d0 + d1) * inverse;
  }
}

// ---------------------------------------------------------------------------
// apply_bits / unpack_rows / packed_embedding: one thread per packed byte
// ---------------------------------------------------------------------------

template <typename T>
__global__ void apply_bits_kernel(const T* __restrict__ values, const uint8_t* __restrict__ packed,
                                  int64_t rows, int64_t columns, T* __restrict__ out) {
  const int64_t stride = (columns + 7) >> 3;
  const int64_t total = rows * stride;
  for (int64_t q = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; q < total;
       q += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = q / stride, byte = q - row * stride;
    const unsigned bits = packed[q];
    const int64_t base = row * columns + byte * 8;
    const int limit = (int)((columns - byte * 8) < 8 ? (columns - byte * 8) : 8);
    for (int b = 0; b < limit; ++b) {
      const float v = DType<T>::load(values + base + b);
      DType<T>::store(out + base + b, v * (((bits >> b) & 1u) ? 1.0f : 0.0f));
    }
  }
}

template <typename T>
__global__ void unpack_rows_kernel(const uint8_t* __restrict__ packed, int64_t rows, int64_t columns,
                                   T* __restrict__ out, int zero_one) {
  const int64_t stride = (columns + 7) >> 3;
  const int64_t total = rows * stride;
  const float low = zero_one ? 0.0f : -1.0f;
  for (int64_t q = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; q < total;
       q += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = q / stride, byte = q - row * stride;
    const unsigned bits = packed[q];
    const int64_t base = row * columns + byte * 8;
    const int limit = (int)((columns - byte * 8) < 8 ? (columns - byte * 8) : 8);
    for (int b = 0; b < limit; ++b)
      DType<T>::store(out + base + b, ((bits >> b) & 1u) ? 1.0f : low);
  }
}

template <typename T>
__global__ void packed_embedding_kernel(const int64_t* __restrict__ ids, int64_t count,
                                        const uint8_t* __restrict__ packed,
                                        const float* __restrict__ scale, int64_t rows,
                                        int64_t columns, T* __restrict__ out, int32_t* bad_id) {
  const int64_t stride = (columns + 7) >> 3;
  const int64_t total = count * stride;
  for (int64_t q = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; q < total;
       q += (int64_t)gridDim.x * blockDim.x) {
    const int64_t index = q / stride, byte = q - index * stride;
    const int64_t row = ids[index];
    const bool ok = row >= 0 && row < rows;
    if (!ok && bad_id) *bad_id = 1;
    const unsigned bits = ok ? packed[row * stride + byte] : 0u;
    const float magnitude = ok ? scale[row] : 0.0f;
    const int64_t base = index * columns + byte * 8;
    const int limit = (int)((columns - byte * 8) < 8 ? (columns - byte * 8) : 8);
    for (int b = 0; b < limit; ++b)
      DType<T>::store(out + base + b, ((bits >> b) & 1u) ? magnitude : -magnitude);
  }
}

// ---------------------------------------------------------------------------
// packed_row_inner: one warp per row, float tolerance (order is not the
// reference's; the result is a float gradient, not an integer state)
// ---------------------------------------------------------------------------

__global__ void __launch_bounds__(256)
packed_row_inner_kernel(const float* __restrict__ matrix, const uint8_t* __restrict__ packed,
                        int64_t rows, int64_t columns, float* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int64_t stride = (columns + 7) >> 3;
  const int64_t full = columns >> 3;
  const float* line = matrix + row * columns;
  const uint8_t* bits = packed + row * stride;
  const bool vector_ok = (columns & 3) == 0 && (reinterpret_cast<uintptr_t>(matrix) & 15) == 0;
  float total = 0.0f;
  for (int64_t byte = lane; byte < full; byte += 32) {
    const unsigned b = bits[byte];
    float v[8];
    if (vector_ok) {
      const float4 lo = *reinterpret_cast<const float4*>(line + byte * 8);
      const float4 hi = *reinterpret_cast<const float4*>(line + byte * 8 + 4);
      v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
      v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
    } else {
      for (int e = 0; e < 8; ++e) v[e] = line[byte * 8 + e];
    }
    float partial = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e) partial += apply_sign(v[e], (b >> e) & 1u);
    total += partial;
  }
  if (lane == 0)
    for (int64_t column = full * 8; column < columns; ++column)
      total += apply_sign(line[column], (bits[full] >> (column - full * 8)) & 1u);
  total = warp_sum(total);
  if (lane == 0) out[row] = total;
}

static inline int grid_for(int64_t items, int threads) {
  int64_t blocks = ceil_div(items, threads);
  const int64_t cap = (int64_t)sm_count() * 32;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace qste

using namespace qste;

extern "C" {

int qste_b200_pack_coordinate(const int8_t* coordinate, int64_t rows, int64_t columns,
                              uint8_t* packed, qste_stream_t stream) {
  if (rows < 0 || columns < 0) return QSTE_ERR_SHAPE;
  if (rows == 0 || columns == 0) return QSTE_OK;
  if (!coordinate || !packed) return QSTE_ERR_NULL;
  const int64_t total = rows * ((columns + 7) / 8);
  if (columns % 64 == 0 && aligned(coordinate, 16) && aligned(packed, 8)) {
    const int64_t groups = rows * (columns / 64);
    pack_bytes_wide_kernel<true><<<grid_for(groups, 256), 256, 0, as_stream(stream)>>>(
        reinterpret_cast<const uint4*>(coordinate), groups, reinterpret_cast<uint2*>(packed));
  } else {
    pack_bytes_kernel<true><<<grid_for(total, 256), 256, 0, as_stream(stream)>>>(
        reinterpret_cast<const uint8_t*>(coordinate), rows, columns, packed);
  }
  note_launches(1);
  return launch_status("pack_coordinate");
}

int qste_b200_pack_bits(const uint8_t* mask, int64_t rows, int64_t columns, uint8_t* packed,
                        qste_stream_t stream) {
  if (rows < 0 || columns < 0) return QSTE_ERR_SHAPE;
  if (rows == 0 || columns == 0) return QSTE_OK;
  if (!mask || !packed) return QSTE_ERR_NULL;
  const int64_t total = rows * ((columns + 7) / 8);
  if (columns % 64 == 0 && aligned(mask, 16) && aligned(packed, 8)) {
    const int64_t groups = rows * (columns / 64);
    pack_bytes_wide_kernel<false><<<grid_for(groups, 256), 256, 0, as_stream(stream)>>>(
        reinterpret_cast<const uint4*>(mask), groups, reinterpret_cast<uint2*>(packed));
  } else {
    pack_bytes_kernel<false><<<grid_for(total, 256), 256, 0, as_stream(stream)>>>(mask, rows, columns,
                                                                                 packed);
  }
  note_launches(1);
  return launch_status("pack_bits");
}

int qste_b200_pack_affine_rows(const void* values, int dtype, int64_t rows, int64_t columns,
                               uint8_t* packed, float* offset, float* scale,
                               qste_stream_t stream) {
  if (rows < 0 || columns < 0) return QSTE_ERR_SHAPE;
  if (rows == 0) return QSTE_OK;
  if (!packed && columns > 0) return QSTE_ERR_NULL;
  if (!values && columns > 0) return QSTE_ERR_NULL;
  if (!offset || !scale) return QSTE_ERR_NULL;
  const size_t element = dtype_size(dtype);
  if (element == 0) return QSTE_ERR_DTYPE;
  const int vector_ok = aligned(values, 16) && ((columns * (int64_t)element) % 16 == 0);
  if (vector_ok && columns > 0) {
    const int blocks = (int)ceil_div(rows, kAsyncWarps * kRowsPerWarp);
    QSTE_DISPATCH_DTYPE(dtype, T,
                        (pack_affine_rows_async_kernel<T><<<blocks, kAsyncWarps * 32, 0, as_stream(stream)>>>(
                            static_cast<const T*>(values), rows, columns, packed, offset, scale)));
    note_launches(1);
    return launch_status("pack_affine_rows");
  }
  const int blocks = (int)ceil_div(rows, kPackWarps * kRowsPerWarp);
  QSTE_DISPATCH_DTYPE(dtype, T,
                      (pack_affine_rows_kernel<T><<<blocks, kPackWarps * 32, 0, as_stream(stream)>>>(
                          static_cast<const T*>(values), rows, columns, packed, offset, scale,
                          vector_ok)));
  note_launches(1);
  return launch_status("pack_affine_rows");
}

int qste_b200_apply_bits(const void* values, int dtype, const uint8_t* packed, int64_t rows,
                         int64_t columns, void* out, qste_stream_t stream) {
  if (rows < 0 || columns < 0) return QSTE_ERR_SHAPE;
  if (rows == 0 || columns == 0) return QSTE_OK;
  if (!values || !packed || !out) return QSTE_ERR_NULL;
  const int64_t total = rows * ((columns + 7) / 8);
  QSTE_DISPATCH_DTYPE(dtype, T,
                      (apply_bits_kernel<T><<<grid_for(total, 256), 256, 0, as_stream(stream)>>>(
                          static_cast<const T*>(values), packed, rows, columns,
                          static_cast<T*>(out))));
  note_launches(1);
  return launch_status("apply_bits");
}

int qste_b200_unpack_rows(const uint8_t* packed, int64_t rows, int64_t columns, void* out,
                          int dtype, int zero_one, qste_stream_t stream) {
  if (rows < 0 || columns < 0) return QSTE_ERR_SHAPE;
  if (rows == 0 || columns == 0) return QSTE_OK;
  if (!packed || !out) return QSTE_ERR_NULL;
  const int64_t total = rows * ((columns + 7) / 8);
  QSTE_DISPATCH_DTYPE(dtype, T,
                      (unpack_rows_kernel<T><<<grid_for(total, 256), 256, 0, as_stream(stream)>>>(
                          packed, rows, columns, static_cast<T*>(out), zero_one)));
  note_launches(1);
  return launch_status("unpack_rows");
}

int qste_b200_packed_row_inner(const float* matrix, const uint8_t* packed, int64_t rows,
                               int64_t columns, float* out, qste_stream_t stream) {
  if (rows < 0 || columns < 0) return QSTE_ERR_SHAPE;
  if (rows == 0) return QSTE_OK;
  if (!out || (columns > 0 && (!matrix || !packed))) return QSTE_ERR_NULL;
  const int warps = 8;
  packed_row_inner_kernel<<<(unsigned)ceil_div(rows, warps), warps * 32, 0, as_stream(stream)>>>(
      matrix, packed, rows, columns, out);
  note_launches(1);
  return launch_status("packed_row_inner");
}

int qste_b200_packed_embedding(const int64_t* ids, int64_t count, const uint8_t* packed,
                               const float* scale, int64_t rows, int64_t columns, void* out,
                               int out_dtype, int32_t* bad_id, qste_stream_t stream) {
  if (count < 0 || rows < 0 || columns < 0) return QSTE_ERR_SHAPE;
  if (count == 0 || columns == 0) return QSTE_OK;
  if (!ids || !packed || !scale || !out) return QSTE_ERR_NULL;
  const int64_t total = count * ((columns + 7) / 8);
  QSTE_DISPATCH_DTYPE(
      out_dtype, T,
      (packed_embedding_kernel<T><<<grid_for(total, 256), 256, 0, as_stream(stream)>>>(
          ids, count, packed, scale, rows, columns, static_cast<T*>(out), bad_id)));
  note_launches(1);
  return launch_status("packed_embedding");
}

}  // extern "C"
