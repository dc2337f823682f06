// Epilogue of the tcgen05 GEMM kernels: one thread owns one output row and handles 32
// consecutive fp32 accumulator columns at a time (the shape `tcgen05.ld.32x32b.x32` returns).
#pragma once

#include "sm100_ptx.cuh"
#include "dp_reduce.h"

namespace elfb {

// D[row, col..col+32) (+)= alpha * v (+ bias); 16-byte vector accesses when the chunk is
// fully inside the matrix, element-wise on the ragged right edge.  With a push target
// (16-bit output only) the finished values are also stored at the same [row, col] of the
// matrix copy inside every peer GPU's inbox: plain stores to peer memory over NVLink.
template <bool OUT_F32, bool ACCUM, bool BIAS>
__device__ __forceinline__ void store_accumulator_chunk(const uint32_t (&v)[32], int row, int col, int M, int N, void* __restrict__ d_ptr,
                                                        long long ldd, const void* __restrict__ bias_ptr, uint32_t fmt, float alpha,
                                                        const PushTarget& push) {
  if (row < M) {
    const bool full_chunk = col + 32 <= N;
    if (OUT_F32) {
      float* dst = reinterpret_cast<float*>(d_ptr) + (long long)row * ldd + col;
      if (full_chunk) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          float4 o;
          o.x = __uint_as_float(v[j]) * alpha;
          o.y = __uint_as_float(v[j + 1]) * alpha;
          o.z = __uint_as_float(v[j + 2]) * alpha;
          o.w = __uint_as_float(v[j + 3]) * alpha;
          if (BIAS) {
            const float* b = reinterpret_cast<const float*>(bias_ptr) + col + j;
            o.x += b[0]; o.y += b[1]; o.z += b[2]; o.w += b[3];
          }
          if (ACCUM) {
            const float4 p = *reinterpret_cast<const float4*>(dst + j);
            o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
          }
          *reinterpret_cast<float4*>(dst + j) = o;
        }
      } else {
        for (int j = 0; j < 32 && col + j < N; ++j) {
          float o = __uint_as_float(v[j]) * alpha;
          if (BIAS) o += reinterpret_cast<const float*>(bias_ptr)[col + j];
          if (ACCUM) o += dst[j];
          dst[j] = o;
        }
      }
    } else {
      // 16-bit output (same format as the operands)
      uint16_t* dst = reinterpret_cast<uint16_t*>(d_ptr) + (long long)row * ldd + col;
      const uint16_t* bias16 = reinterpret_cast<const uint16_t*>(bias_ptr);
      auto to_f = [&](uint16_t h) -> float {
        return fmt == 1u ? __bfloat162float(__ushort_as_bfloat16(h)) : __half2float(__ushort_as_half(h));
      };
      auto pack2 = [&](float a, float b) -> uint32_t { return fmt == 1u ? pack_bf16x2(a, b) : pack_f16x2(a, b); };
      if (full_chunk) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          float f[8];
#pragma unroll
          for (int t = 0; t < 8; ++t) f[t] = __uint_as_float(v[j + t]) * alpha;
          if (BIAS) {
            const uint4 bq = *reinterpret_cast<const uint4*>(bias16 + col + j);
            const uint32_t bw[4] = {bq.x, bq.y, bq.z, bq.w};
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              f[2 * t] += to_f(uint16_t(bw[t] & 0xffff));
              f[2 * t + 1] += to_f(uint16_t(bw[t] >> 16));
            }
          }
          if (ACCUM) {
            const uint4 pq = *reinterpret_cast<const uint4*>(dst + j);
            const uint32_t pw[4] = {pq.x, pq.y, pq.z, pq.w};
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              f[2 * t] += to_f(uint16_t(pw[t] & 0xffff));
              f[2 * t + 1] += to_f(uint16_t(pw[t] >> 16));
            }
          }
          uint4 o;
          o.x = pack2(f[0], f[1]);
          o.y = pack2(f[2], f[3]);
          o.z = pack2(f[4], f[5]);
          o.w = pack2(f[6], f[7]);
          *reinterpret_cast<uint4*>(dst + j) = o;
          for (int p = 0; p < push.n_peers; ++p)
            *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(push.peer_out[p]) + (long long)row * ldd + col + j) = o;
        }
      } else {
        for (int j = 0; j < 32 && col + j < N; ++j) {
          float o = __uint_as_float(v[j]) * alpha;
          if (BIAS) o += to_f(bias16[col + j]);
          if (ACCUM) o += to_f(dst[j]);
          const uint16_t h = uint16_t(pack2(o, 0.f) & 0xffff);
          dst[j] = h;
          for (int p = 0; p < push.n_peers; ++p) (reinterpret_cast<uint16_t*>(push.peer_out[p]) + (long long)row * ldd + col)[j] = h;
        }
      }
    }
  }
}

}  // namespace elfb
