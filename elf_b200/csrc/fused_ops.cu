// Bandwidth-bound kernels for sm_100a: RMSNorm, RoPE, SwiGLU, cross-entropy, embedding,
// AdamW.  All move 16 bytes per thread per access and keep fp32 math in registers; the
// roofline for each is HBM traffic only.
#include "fused_ops.h"

#include <cuda_bf16.h>

#include <cstdlib>

namespace elfb {

namespace {

struct alignas(16) Bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const Bf16x8& p, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ Bf16x8 pack8(const float (&f)[8]) {
  Bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; every thread gets the result.  `red` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nwarps ? red[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nwarps ? red[lane] : -INFINITY;
  return warp_max(t);
}

// ------------------------------------------------------------------------------ RMSNorm
// One block per row, the row held in registers.  Rows of up to 4096 elements run on 128-thread
// blocks (four 16-byte vectors per thread): twice as many resident blocks per SM as with 256
// threads, so twice as many bytes in flight per SM, and half as many warps in the block-wide sum.
constexpr int RMS_MAX_VEC = 4;  // rows up to RMS_THREADS*4*8 elements stay in registers (4096 / 8192)

template <bool RESIDUAL, int RMS_THREADS>
__global__ void __launch_bounds__(RMS_THREADS) rmsnorm_fwd_kernel(const Bf16x8* __restrict__ x, const Bf16x8* __restrict__ res,
                                                                  const Bf16x8* __restrict__ w, Bf16x8* __restrict__ y,
                                                                  Bf16x8* __restrict__ h, float* __restrict__ rstd, int dim8,
                                                                  float inv_dim, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const Bf16x8* xr = x + row * dim8;
  float vals[RMS_MAX_VEC][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < RMS_MAX_VEC; ++it) {
    const int i = threadIdx.x + it * RMS_THREADS;
    if (i < dim8) {
      unpack8(xr[i], vals[it]);
      if (RESIDUAL) {
        float r[8];
        unpack8(res[row * dim8 + i], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) vals[it][j] += r[j];
        const Bf16x8 hv = pack8(vals[it]);
        h[row * dim8 + i] = hv;
        unpack8(hv, vals[it]);  // normalise exactly what later passes will read back
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += vals[it][j] * vals[it][j];
    }
  }
  for (int i = threadIdx.x + RMS_MAX_VEC * RMS_THREADS; i < dim8; i += RMS_THREADS) {  // very wide rows
    float t[8];
    unpack8(xr[i], t);
    if (RESIDUAL) {
      float r[8];
      unpack8(res[row * dim8 + i], r);
      for (int j = 0; j < 8; ++j) t[j] += r[j];
      const Bf16x8 hv = pack8(t);
      h[row * dim8 + i] = hv;
      unpack8(hv, t);
    }
    for (int j = 0; j < 8; ++j) ss += t[j] * t[j];
  }
  ss = block_sum(ss, red);
  const float rs = rsqrtf(ss * inv_dim + eps);
  if (threadIdx.x == 0) rstd[row] = rs;
#pragma unroll
  for (int it = 0; it < RMS_MAX_VEC; ++it) {
    const int i = threadIdx.x + it * RMS_THREADS;
    if (i < dim8) {
      float wv[8], o[8];
      unpack8(w[i], wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = vals[it][j] * rs * wv[j];
      y[row * dim8 + i] = pack8(o);
    }
  }
  for (int i = threadIdx.x + RMS_MAX_VEC * RMS_THREADS; i < dim8; i += RMS_THREADS) {
    float t[8], wv[8], o[8];
    unpack8(RESIDUAL ? h[row * dim8 + i] : xr[i], t);
    unpack8(w[i], wv);
    for (int j = 0; j < 8; ++j) o[j] = t[j] * rs * wv[j];
    y[row * dim8 + i] = pack8(o);
  }
}

// Backward in two bandwidth-shaped kernels.
//   dx:  one block per row, the row lives in registers (same shape as the forward).
//   dw:  grid (dim/256 column slabs, RMS_DW_SPLITS row groups); a block's 256 threads form
//        32 column groups (8 columns each) x 8 row lanes and walk the rows of their group;
//        the 8 lanes are summed through shared memory and written as one partial row.
constexpr int RMS_DW_SPLITS = 64;

template <bool DRES, int RMS_THREADS>
__global__ void __launch_bounds__(RMS_THREADS) rmsnorm_bwd_dx_kernel(const Bf16x8* __restrict__ dy, const Bf16x8* __restrict__ x,
                                                                     const Bf16x8* __restrict__ w, const float* __restrict__ rstd,
                                                                     const Bf16x8* __restrict__ dres, Bf16x8* __restrict__ dx,
                                                                     int dim8, float inv_dim) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const float rs = rstd[row];
  float xv[RMS_MAX_VEC][8], gv[RMS_MAX_VEC][8];
  float dot = 0.f;
#pragma unroll
  for (int it = 0; it < RMS_MAX_VEC; ++it) {
    const int i = threadIdx.x + it * RMS_THREADS;
    if (i < dim8) {
      float wv[8];
      unpack8(x[row * dim8 + i], xv[it]);
      unpack8(dy[row * dim8 + i], gv[it]);
      unpack8(w[i], wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        gv[it][j] *= wv[j];
        dot += gv[it][j] * xv[it][j];
      }
    }
  }
  dot = block_sum(dot, red);
  const float c = dot * inv_dim * rs * rs * rs;
#pragma unroll
  for (int it = 0; it < RMS_MAX_VEC; ++it) {
    const int i = threadIdx.x + it * RMS_THREADS;
    if (i < dim8) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = gv[it][j] * rs - xv[it][j] * c;
      if (DRES) {
        float r[8];
        unpack8(dres[row * dim8 + i], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += r[j];
      }
      dx[row * dim8 + i] = pack8(o);
    }
  }
}

__global__ void __launch_bounds__(256) rmsnorm_bwd_dw_kernel(const Bf16x8* __restrict__ dy, const Bf16x8* __restrict__ x,
                                                             const float* __restrict__ rstd, float* __restrict__ dw_partial, int rows,
                                                             int dim8) {
  __shared__ float red[8][32][8];
  const int cg = threadIdx.x & 31;   // column group within the slab
  const int lane_r = threadIdx.x >> 5;  // row lane 0..7
  const int col8 = blockIdx.x * 32 + cg;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col8 < dim8) {
    for (long long row = (long long)blockIdx.y * 8 + lane_r; row < rows; row += (long long)gridDim.y * 8) {
      float a[8], b[8];
      unpack8(dy[row * dim8 + col8], a);
      unpack8(x[row * dim8 + col8], b);
      const float rs = rstd[row];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += a[j] * b[j] * rs;
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[lane_r][cg][j] = acc[j];
  __syncthreads();
  if (lane_r == 0 && col8 < dim8) {
    float s[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      s[j] = 0.f;
#pragma unroll
      for (int r = 0; r < 8; ++r) s[j] += red[r][cg][j];
    }
    float* dst = dw_partial + ((long long)blockIdx.y * dim8 + col8) * 8;
    *reinterpret_cast<float4*>(dst) = make_float4(s[0], s[1], s[2], s[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(s[4], s[5], s[6], s[7]);
  }
}

__global__ void colsum_kernel(const float* __restrict__ partial, float* __restrict__ out, int nblocks, int dim, bool accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= dim) return;
  float s = 0.f;
  for (int b = 0; b < nblocks; ++b) s += partial[(long long)b * dim + c];
  out[c] = accumulate ? out[c] + s : s;
}

// Persistent variants for the common widths (dim = 256 * VPT * 8: 2048, 4096, 8192).  A block of
// 256 threads walks rows blockIdx.x, blockIdx.x + gridDim.x, ...; thread t always owns the same
// VPT 16-byte column groups (t, t + 256, ...), so the gain stays in registers, the loads of the
// next row are issued before the current row is reduced (reads and writes of different rows
// overlap instead of alternating), and - in the backward - the gain's gradient is accumulated
// in registers over all rows of the block: one pass over dy and x instead of two.
template <bool RESIDUAL, int VPT>
__global__ void __launch_bounds__(256) rmsnorm_fwd_persistent_kernel(const Bf16x8* __restrict__ x, const Bf16x8* __restrict__ res,
                                                                     const Bf16x8* __restrict__ w, Bf16x8* __restrict__ y,
                                                                     Bf16x8* __restrict__ h, float* __restrict__ rstd, int rows,
                                                                     float inv_dim, float eps) {
  constexpr int DIM8 = 256 * VPT;
  __shared__ float red[32];
  float wv[VPT][8];
#pragma unroll
  for (int v = 0; v < VPT; ++v) unpack8(w[threadIdx.x + v * 256], wv[v]);
  long long row = blockIdx.x;
  Bf16x8 nx[VPT], nr[VPT];
  if (row < rows) {
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      nx[v] = x[row * DIM8 + threadIdx.x + v * 256];
      if (RESIDUAL) nr[v] = res[row * DIM8 + threadIdx.x + v * 256];
    }
  }
  for (; row < rows; row += gridDim.x) {
    float vals[VPT][8];
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      unpack8(nx[v], vals[v]);
      if (RESIDUAL) {
        float r[8];
        unpack8(nr[v], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) vals[v][j] += r[j];
      }
    }
    const long long next = row + gridDim.x;
    if (next < rows) {  // prefetch the next row of this block
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        nx[v] = x[next * DIM8 + threadIdx.x + v * 256];
        if (RESIDUAL) nr[v] = res[next * DIM8 + threadIdx.x + v * 256];
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      if (RESIDUAL) {
        const Bf16x8 hv = pack8(vals[v]);
        h[row * DIM8 + threadIdx.x + v * 256] = hv;
        unpack8(hv, vals[v]);  // normalise exactly what later passes will read back
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += vals[v][j] * vals[v][j];
    }
    ss = block_sum(ss, red);
    const float rs = rsqrtf(ss * inv_dim + eps);
    if (threadIdx.x == 0) rstd[row] = rs;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = vals[v][j] * rs * wv[v][j];
      y[row * DIM8 + threadIdx.x + v * 256] = pack8(o);
    }
  }
}

template <bool DRES, int VPT>
__global__ void __launch_bounds__(256) rmsnorm_bwd_persistent_kernel(const Bf16x8* __restrict__ dy, const Bf16x8* __restrict__ x,
                                                                     const Bf16x8* __restrict__ w, const float* __restrict__ rstd,
                                                                     const Bf16x8* __restrict__ dres, Bf16x8* __restrict__ dx,
                                                                     float* __restrict__ dw_partial, int rows, float inv_dim) {
  constexpr int DIM8 = 256 * VPT;
  __shared__ float red[32];
  float wv[VPT][8], dwacc[VPT][8];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    unpack8(w[threadIdx.x + v * 256], wv[v]);
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[v][j] = 0.f;
  }
  long long row = blockIdx.x;
  Bf16x8 ng[VPT], nx[VPT], nr[VPT];
  if (row < rows) {
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      ng[v] = dy[row * DIM8 + threadIdx.x + v * 256];
      nx[v] = x[row * DIM8 + threadIdx.x + v * 256];
      if (DRES) nr[v] = dres[row * DIM8 + threadIdx.x + v * 256];
    }
  }
  for (; row < rows; row += gridDim.x) {
    float gv[VPT][8], xv[VPT][8], rv[VPT][8];
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      unpack8(ng[v], gv[v]);
      unpack8(nx[v], xv[v]);
      if (DRES) unpack8(nr[v], rv[v]);
    }
    const float rs = rstd[row];
    const long long next = row + gridDim.x;
    if (next < rows) {
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        ng[v] = dy[next * DIM8 + threadIdx.x + v * 256];
        nx[v] = x[next * DIM8 + threadIdx.x + v * 256];
        if (DRES) nr[v] = dres[next * DIM8 + threadIdx.x + v * 256];
      }
    }
    float dot = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        dwacc[v][j] += gv[v][j] * xv[v][j] * rs;
        gv[v][j] *= wv[v][j];
        dot += gv[v][j] * xv[v][j];
      }
    }
    dot = block_sum(dot, red);
    const float c = dot * inv_dim * rs * rs * rs;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j] = gv[v][j] * rs - xv[v][j] * c;
        if (DRES) o[j] += rv[v][j];
      }
      dx[row * DIM8 + threadIdx.x + v * 256] = pack8(o);
    }
  }
  // one partial row per block: dw_partial[blockIdx.x][dim]
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    float* dst = dw_partial + ((long long)blockIdx.x * DIM8 + threadIdx.x + v * 256) * 8;
    *reinterpret_cast<float4*>(dst) = make_float4(dwacc[v][0], dwacc[v][1], dwacc[v][2], dwacc[v][3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(dwacc[v][4], dwacc[v][5], dwacc[v][6], dwacc[v][7]);
  }
}

// Column sums of a tall `partial[nrows][dim]` (one row per block of the persistent backward): a block
// of 256 threads covers 32 columns with 8 row lanes, so the few hundred rows are read by
// dim/32 blocks in parallel instead of one thread walking each column.  OUT is float
// (written or accumulated) or bf16 (a gradient buffer: always accumulated, in fp32).
template <typename OUT>
__global__ void __launch_bounds__(256) colsum_tall_kernel(const float* __restrict__ partial, OUT* __restrict__ out, int nrows, int dim, bool accumulate) {
  __shared__ float red[8][32];
  const int col = blockIdx.x * 32 + (threadIdx.x & 31);
  const int lane_r = threadIdx.x >> 5;
  float s = 0.f;
  if (col < dim)
    for (int r = lane_r; r < nrows; r += 8) s += partial[(long long)r * dim + col];
  red[lane_r][threadIdx.x & 31] = s;
  __syncthreads();
  if (lane_r == 0 && col < dim) {
    float t = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) t += red[r][threadIdx.x];
    if constexpr (sizeof(OUT) == 2) {
      out[col] = __float2bfloat16_rn(__bfloat162float(out[col]) + t);
    } else {
      out[col] = accumulate ? out[col] + t : t;
    }
  }
}

// Same reduction as colsum_kernel, added into a bf16 vector (a parameter's gradient buffer) in fp32.
__global__ void colsum_add_bf16_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, int nblocks, int dim) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= dim) return;
  float s = __bfloat162float(out[c]);
  for (int b = 0; b < nblocks; ++b) s += partial[(long long)b * dim + c];
  out[c] = __float2bfloat16_rn(s);
}

// dqkv[b, s, :, :] <- (dq[b, s, hq heads], dk[b, s, hkv heads], dv[b, s, hkv heads]): one pass that packs the three
// gradients an attention backward returns (any strides with a contiguous head dimension) into the
// layout of the fused QKV projection.  One thread moves 16 bytes.
// The same packing with RoPE's backward applied on the way: query and key heads are rotated by
// -angle(position).  One thread moves the two 16-byte groups (i, i + head_dim/2) of a rotation pair.
__global__ void __launch_bounds__(256) pack_qkv_grad_rope_kernel(const __nv_bfloat16* __restrict__ dq, const __nv_bfloat16* __restrict__ dk,
                                                                 const __nv_bfloat16* __restrict__ dv, __nv_bfloat16* __restrict__ out,
                                                                 const float* __restrict__ cos_t, const float* __restrict__ sin_t, long long total,
                                                                 int seq, int hq, int hkv, int half, long long q_sb, long long q_ss, long long q_sh,
                                                                 long long k_sb, long long k_ss, long long k_sh, long long v_sb, long long v_ss,
                                                                 long long v_sh) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int heads = hq + 2 * hkv;
  const int vph = half / 8;  // 16-byte groups per half head
  const int v = idx % vph;
  const int h = (idx / vph) % heads;
  const long long bs = idx / ((long long)vph * heads);
  const long long s_ = bs % seq, b = bs / seq;
  const __nv_bfloat16* src;
  if (h < hq) src = dq + b * q_sb + s_ * q_ss + h * q_sh;
  else if (h < hq + hkv) src = dk + b * k_sb + s_ * k_ss + (h - hq) * k_sh;
  else src = dv + b * v_sb + s_ * v_ss + (h - hq - hkv) * v_sh;
  __nv_bfloat16* dst = out + (bs * heads + h) * (2LL * half);
  const Bf16x8 lo = *reinterpret_cast<const Bf16x8*>(src + v * 8), hi = *reinterpret_cast<const Bf16x8*>(src + half + v * 8);
  if (h >= hq + hkv) {  // value heads: no rotation
    *reinterpret_cast<Bf16x8*>(dst + v * 8) = lo;
    *reinterpret_cast<Bf16x8*>(dst + half + v * 8) = hi;
    return;
  }
  float a[8], bb[8], oa[8], ob[8];
  unpack8(lo, a);
  unpack8(hi, bb);
  const float4* c4 = reinterpret_cast<const float4*>(cos_t + s_ * half + v * 8);
  const float4* s4 = reinterpret_cast<const float4*>(sin_t + s_ * half + v * 8);
  const float4 c0 = c4[0], c1 = c4[1], s0 = s4[0], s1 = s4[1];
  const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float sj = -sn[j];  // backward of a rotation is the rotation by the opposite angle
    oa[j] = a[j] * cs[j] - bb[j] * sj;
    ob[j] = bb[j] * cs[j] + a[j] * sj;
  }
  *reinterpret_cast<Bf16x8*>(dst + v * 8) = pack8(oa);
  *reinterpret_cast<Bf16x8*>(dst + half + v * 8) = pack8(ob);
}

__global__ void __launch_bounds__(256) pack_qkv_grad_kernel(const Bf16x8* __restrict__ dq, const Bf16x8* __restrict__ dk, const Bf16x8* __restrict__ dv,
                                                            Bf16x8* __restrict__ out, long long total, int seq, int hq, int hkv, int d8,
                                                            long long q_sb, long long q_ss, long long q_sh, long long k_sb, long long k_ss,
                                                            long long k_sh, long long v_sb, long long v_ss, long long v_sh) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int heads = hq + 2 * hkv;
  const int c = idx % d8;
  const int h = (idx / d8) % heads;
  const long long bs = idx / ((long long)d8 * heads);
  const long long s_ = bs % seq, b = bs / seq;
  // strides are in elements of 8 bf16
  if (h < hq) out[idx] = dq[b * q_sb + s_ * q_ss + h * q_sh + c];
  else if (h < hq + hkv) out[idx] = dk[b * k_sb + s_ * k_ss + (h - hq) * k_sh + c];
  else out[idx] = dv[b * v_sb + s_ * v_ss + (h - hq - hkv) * v_sh + c];
}

// out[i] += res[i] (bf16, fp32 add): the residual connection after a projection
__global__ void residual_add_kernel(Bf16x8* __restrict__ out, const Bf16x8* __restrict__ res, long long n8) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  float a[8], b[8];
  unpack8(out[i], a);
  unpack8(res[i], b);
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] += b[j];
  out[i] = pack8(a);
}

// ------------------------------------------------------------------------------ RoPE
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                            long long total, int row_stride, int n_rot_heads, int half, int seq_len, float sign) {
  // one thread rotates 8 consecutive pairs (i, i + half) of one head
  const int vec_per_head = half / 8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int v = idx % vec_per_head;
  const int head = (idx / vec_per_head) % n_rot_heads;
  const long long row = idx / ((long long)vec_per_head * n_rot_heads);
  const int pos = row % seq_len;
  __nv_bfloat16* base = x + row * row_stride + head * (2 * half) + v * 8;
  Bf16x8 lo = *reinterpret_cast<Bf16x8*>(base), hi = *reinterpret_cast<Bf16x8*>(base + half);
  float a[8], b[8], oa[8], ob[8];
  unpack8(lo, a);
  unpack8(hi, b);
  const float4* c4 = reinterpret_cast<const float4*>(cos_t + (long long)pos * half + v * 8);
  const float4* s4 = reinterpret_cast<const float4*>(sin_t + (long long)pos * half + v * 8);
  const float4 c0 = c4[0], c1 = c4[1], s0 = s4[0], s1 = s4[1];
  const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float s = sn[j] * sign;
    oa[j] = a[j] * cs[j] - b[j] * s;
    ob[j] = b[j] * cs[j] + a[j] * s;
  }
  *reinterpret_cast<Bf16x8*>(base) = pack8(oa);
  *reinterpret_cast<Bf16x8*>(base + half) = pack8(ob);
}

// ------------------------------------------------------------------------------ SwiGLU
__global__ void swiglu_fwd_kernel(const Bf16x8* __restrict__ gu, Bf16x8* __restrict__ out, long long total, int f8) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long row = idx / f8;
  const int c = idx % f8;
  float g[8], u[8], o[8];
  unpack8(gu[row * 2 * f8 + c], g);
  unpack8(gu[row * 2 * f8 + f8 + c], u);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
  out[idx] = pack8(o);
}
__global__ void swiglu_bwd_kernel(const Bf16x8* __restrict__ dout, const Bf16x8* __restrict__ gu, Bf16x8* __restrict__ dgu,
                                  long long total, int f8) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long row = idx / f8;
  const int c = idx % f8;
  float g[8], u[8], d[8], dg[8], du[8];
  unpack8(gu[row * 2 * f8 + c], g);
  unpack8(gu[row * 2 * f8 + f8 + c], u);
  unpack8(dout[idx], d);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float sg = 1.f / (1.f + __expf(-g[j]));
    const float silu = g[j] * sg;
    dg[j] = d[j] * u[j] * (sg + silu * (1.f - sg));
    du[j] = d[j] * silu;
  }
  dgu[row * 2 * f8 + c] = pack8(dg);
  dgu[row * 2 * f8 + f8 + c] = pack8(du);
}

// ------------------------------------------------------------------------------ cross entropy
constexpr int CE_THREADS = 1024;

__global__ void __launch_bounds__(CE_THREADS) ce_fwd_kernel(const __nv_bfloat16* __restrict__ logits,
                                                            const int64_t* __restrict__ targets, float* __restrict__ loss,
                                                            float* __restrict__ lse_out, int vocab, long long ld,
                                                            int64_t ignore_index) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* lr = logits + row * ld;
  const int v8 = vocab / 8;
  // online softmax: running max m and sum s of exp(x - m)
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < v8; i += CE_THREADS) {
    float f[8];
    unpack8(reinterpret_cast<const Bf16x8*>(lr)[i], f);
    float cm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) cm = fmaxf(cm, f[j]);
    const float nm = fmaxf(m, cm);
    float add = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) add += __expf(f[j] - nm);
    s = s * __expf(m - nm) + add;
    m = nm;
  }
  for (int i = v8 * 8 + threadIdx.x; i < vocab; i += CE_THREADS) {
    const float f = __bfloat162float(lr[i]);
    const float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
  }
  const float gm = block_max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum(s, red);
  if (threadIdx.x == 0) {
    const float lse = gm + logf(gs);
    lse_out[row] = lse;
    const int64_t t = targets[row];
    loss[row] = (t == ignore_index || t < 0 || t >= vocab) ? 0.f : lse - __bfloat162float(lr[t]);
  }
}

__global__ void __launch_bounds__(CE_THREADS) ce_bwd_kernel(const __nv_bfloat16* __restrict__ logits,
                                                            __nv_bfloat16* __restrict__ dlogits,
                                                            const int64_t* __restrict__ targets, const float* __restrict__ lse,
                                                            const float* __restrict__ gscale, float scale, int vocab,
                                                            long long ld, int64_t ignore_index) {
  const long long row = blockIdx.x;
  const __nv_bfloat16* lr = logits + row * ld;
  __nv_bfloat16* dr = dlogits + row * ld;
  const int64_t t = targets[row];
  const bool ignored = (t == ignore_index || t < 0 || t >= vocab);
  const float g = ignored ? 0.f : (gscale ? gscale[0] : 1.f) * scale;
  const float l = lse[row];
  const int v8 = vocab / 8;
  for (int i = threadIdx.x; i < v8; i += CE_THREADS) {
    float f[8];
    unpack8(reinterpret_cast<const Bf16x8*>(lr)[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float p = __expf(f[j] - l);
      f[j] = (p - ((long long)i * 8 + j == t ? 1.f : 0.f)) * g;
    }
    reinterpret_cast<Bf16x8*>(dr)[i] = pack8(f);
  }
  for (int i = v8 * 8 + threadIdx.x; i < vocab; i += CE_THREADS) {
    const float p = __expf(__bfloat162float(lr[i]) - l);
    dr[i] = __float2bfloat16((p - (i == t ? 1.f : 0.f)) * g);
  }
}

// Cross entropy over the vocabulary in chunks: the LM head's logits never exist as a whole.
// `logits` holds the columns [col0, col0 + width) of every row.  The statistics kernel folds the
// chunk into the running (max, sum of exp, target logit) of each row; once all chunks are in,
// lse = max + log(sum) and loss = lse - target logit.  The gradient kernel turns a (recomputed)
// chunk into (softmax - onehot) * scale in place.
__global__ void __launch_bounds__(CE_THREADS) ce_chunk_stats_kernel(const __nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                                                                    float* __restrict__ run_max, float* __restrict__ run_sum,
                                                                    float* __restrict__ tgt_logit, int width, long long ld, long long col0,
                                                                    bool first) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* lr = logits + row * ld;
  const int v8 = width / 8;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < v8; i += CE_THREADS) {
    float f[8];
    unpack8(reinterpret_cast<const Bf16x8*>(lr)[i], f);
    float cm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) cm = fmaxf(cm, f[j]);
    const float nm = fmaxf(m, cm);
    float add = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) add += __expf(f[j] - nm);
    s = s * __expf(m - nm) + add;
    m = nm;
  }
  for (int i = v8 * 8 + threadIdx.x; i < width; i += CE_THREADS) {
    const float f = __bfloat162float(lr[i]);
    const float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
  }
  const float gm = block_max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum(s, red);
  if (threadIdx.x == 0) {
    const float pm = first ? -INFINITY : run_max[row];
    const float ps = first ? 0.f : run_sum[row];
    const float nm = fmaxf(pm, gm);
    run_sum[row] = (pm == -INFINITY ? 0.f : ps * __expf(pm - nm)) + gs * __expf(gm - nm);
    run_max[row] = nm;
    const long long t = targets[row] - col0;
    if (first) tgt_logit[row] = 0.f;
    if (t >= 0 && t < width) tgt_logit[row] = __bfloat162float(lr[t]);
  }
}

__global__ void __launch_bounds__(CE_THREADS) ce_chunk_grad_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                                                                   const float* __restrict__ lse, const float* __restrict__ gscale, float scale,
                                                                   int width, long long ld, long long col0, long long vocab,
                                                                   int64_t ignore_index) {
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const int64_t t = targets[row];
  const bool ignored = (t == ignore_index || t < 0 || t >= vocab);
  const float g = ignored ? 0.f : (gscale ? gscale[0] : 1.f) * scale;
  const float l = lse[row];
  const long long tl = t - col0;  // target column inside this chunk, if any
  const int v8 = width / 8;
  for (int i = threadIdx.x; i < v8; i += CE_THREADS) {
    float f[8];
    unpack8(reinterpret_cast<const Bf16x8*>(lr)[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float p = __expf(f[j] - l);
      f[j] = (p - ((long long)i * 8 + j == tl ? 1.f : 0.f)) * g;
    }
    reinterpret_cast<Bf16x8*>(lr)[i] = pack8(f);
  }
  for (int i = v8 * 8 + threadIdx.x; i < width; i += CE_THREADS) {
    const float p = __expf(__bfloat162float(lr[i]) - l);
    lr[i] = __float2bfloat16((p - (i == tl ? 1.f : 0.f)) * g);
  }
}

// ------------------------------------------------------------------------------ embedding
// Error word shared with the GEMM / attention kernels (sm100_ptx.cuh): status[0] = code, [1] = where, [2..3] = detail.
constexpr int kStatusOk = 0, kStatusBadIndex = 4;
__device__ __forceinline__ void report_error(int* status, int code, int where, int a, int b) {
  if (status != nullptr && atomicCAS(status, kStatusOk, code) == kStatusOk) {
    status[1] = where;
    status[2] = a;
    status[3] = b;
  }
}

// A token id outside [0, vocab) reads nothing: its output row is zero, its gradient is dropped, and
// the first such id is recorded in the status word (code 4; where = 1 forward, 2 backward;
// detail = row, id), which the optimizer step and the next pipeline step turn into an exception.
__global__ void embedding_fwd_kernel(const Bf16x8* __restrict__ table, const int64_t* __restrict__ ids, Bf16x8* __restrict__ out,
                                     long long total, int dim8, long long vocab, int* __restrict__ status) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long row = idx / dim8;
  const int c = idx % dim8;
  const int64_t id = ids[row];
  if (id < 0 || id >= vocab) {
    if (c == 0) report_error(status, kStatusBadIndex, 1, (int)row, (int)id);
    const float zero[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    out[idx] = pack8(zero);
    return;
  }
  out[idx] = table[id * dim8 + c];
}
template <bool F32>
__global__ void embedding_bwd_kernel(const __nv_bfloat162* __restrict__ dout, const int64_t* __restrict__ ids, void* __restrict__ dtable,
                                     long long total, int dim2, long long vocab, int* __restrict__ status) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long row = idx / dim2;
  const int c = idx % dim2;
  const int64_t id = ids[row];
  if (id < 0 || id >= vocab) {
    if (c == 0) report_error(status, kStatusBadIndex, 2, (int)row, (int)id);
    return;
  }
  const __nv_bfloat162 g = dout[idx];
  if (F32) {
    float* d = reinterpret_cast<float*>(dtable) + (id * dim2 + c) * 2;
    const float2 f = __bfloat1622float2(g);
    atomicAdd(d, f.x);
    atomicAdd(d + 1, f.y);
  } else {
    atomicAdd(reinterpret_cast<__nv_bfloat162*>(dtable) + id * dim2 + c, g);
  }
}

// Deterministic embedding backward: `sorted_ids` are the token ids in ascending order and
// `perm[k]` the row of `dout` that sorted position k came from (a stable sort).  Block k owns
// the run of equal ids that starts at position k (blocks in the middle of a run exit), sums the
// rows of that run in order in fp32 and adds the sum to the token's row of `grad` - straight
// into the parameter's gradient buffer, no dense temporary, no atomics.
template <bool GRAD_F32>
__global__ void __launch_bounds__(256) embedding_bwd_sorted_kernel(const Bf16x8* __restrict__ dout, const int64_t* __restrict__ sorted_ids,
                                                                   const int64_t* __restrict__ perm, void* __restrict__ grad, int rows,
                                                                   int dim8, long long vocab) {
  const int k = blockIdx.x;
  const int64_t token = sorted_ids[k];
  if (k > 0 && sorted_ids[k - 1] == token) return;  // not the head of its run
  if (token < 0 || token >= vocab) return;          // padding / ignored ids carry no gradient
  int len = 1;
  while (k + len < rows && sorted_ids[k + len] == token) ++len;
  for (int c = threadIdx.x; c < dim8; c += blockDim.x) {
    float acc[8];
    if (GRAD_F32) {
      const float4* g = reinterpret_cast<const float4*>(grad) + ((long long)token * dim8 + c) * 2;
      const float4 a = g[0], b = g[1];
      acc[0] = a.x; acc[1] = a.y; acc[2] = a.z; acc[3] = a.w; acc[4] = b.x; acc[5] = b.y; acc[6] = b.z; acc[7] = b.w;
    } else {
      unpack8(reinterpret_cast<const Bf16x8*>(grad)[(long long)token * dim8 + c], acc);
    }
    for (int j = 0; j < len; ++j) {
      float v[8];
      unpack8(dout[(long long)perm[k + j] * dim8 + c], v);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += v[e];
    }
    if (GRAD_F32) {
      float4* g = reinterpret_cast<float4*>(grad) + ((long long)token * dim8 + c) * 2;
      g[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      g[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    } else {
      reinterpret_cast<Bf16x8*>(grad)[(long long)token * dim8 + c] = pack8(acc);
    }
  }
}

// ------------------------------------------------------------------------------ AdamW
template <bool GRAD_F32>
__global__ void adamw_kernel(Bf16x8* __restrict__ p, const void* __restrict__ grad, float* __restrict__ master,
                             float* __restrict__ m, float* __restrict__ v, long long n8, long long n, float lr, float b1,
                             float b2, float eps, float decay, float inv_bc1, float inv_bc2, float gscale,
                             const int* __restrict__ status) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  // a kernel of this step gave up on a bounded wait: the gradients cannot be trusted
  if (status != nullptr && *status != 0) return;
  const long long base = i * 8;
  float g[8];
  if (base + 8 <= n) {
    if (GRAD_F32) {
      const float4 a = reinterpret_cast<const float4*>(grad)[2 * i], b = reinterpret_cast<const float4*>(grad)[2 * i + 1];
      g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w; g[4] = b.x; g[5] = b.y; g[6] = b.z; g[7] = b.w;
    } else {
      unpack8(reinterpret_cast<const Bf16x8*>(grad)[i], g);
    }
    float4 w0 = reinterpret_cast<float4*>(master)[2 * i], w1 = reinterpret_cast<float4*>(master)[2 * i + 1];
    float4 m0 = reinterpret_cast<float4*>(m)[2 * i], m1 = reinterpret_cast<float4*>(m)[2 * i + 1];
    float4 v0 = reinterpret_cast<float4*>(v)[2 * i], v1 = reinterpret_cast<float4*>(v)[2 * i + 1];
    float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
    float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = g[j] * gscale;
      mm[j] = b1 * mm[j] + (1.f - b1) * gj;
      vv[j] = b2 * vv[j] + (1.f - b2) * gj * gj;
      const float upd = (mm[j] * inv_bc1) / (sqrtf(vv[j] * inv_bc2) + eps);
      w[j] = w[j] * decay - lr * upd;
    }
    reinterpret_cast<float4*>(master)[2 * i] = make_float4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<float4*>(master)[2 * i + 1] = make_float4(w[4], w[5], w[6], w[7]);
    reinterpret_cast<float4*>(m)[2 * i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(m)[2 * i + 1] = make_float4(mm[4], mm[5], mm[6], mm[7]);
    reinterpret_cast<float4*>(v)[2 * i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    reinterpret_cast<float4*>(v)[2 * i + 1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
    p[i] = pack8(w);
  } else {
    for (long long k = base; k < n; ++k) {  // ragged tail
      const float gj = (GRAD_F32 ? reinterpret_cast<const float*>(grad)[k]
                                 : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(grad)[k])) * gscale;
      const float mk = b1 * m[k] + (1.f - b1) * gj;
      const float vk = b2 * v[k] + (1.f - b2) * gj * gj;
      const float wk = master[k] * decay - lr * (mk * inv_bc1) / (sqrtf(vk * inv_bc2) + eps);
      m[k] = mk; v[k] = vk; master[k] = wk;
      reinterpret_cast<__nv_bfloat16*>(p)[k] = __float2bfloat16(wk);
    }
  }
}

__global__ void scale_bf16_kernel(Bf16x8* __restrict__ x, long long n8, long long n, float a) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  if (i * 8 + 8 <= n) {
    float f[8];
    unpack8(x[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] *= a;
    x[i] = pack8(f);
  } else {
    __nv_bfloat16* t = reinterpret_cast<__nv_bfloat16*>(x);
    for (long long k = i * 8; k < n; ++k) t[k] = __float2bfloat16(__bfloat162float(t[k]) * a);
  }
}

inline int blocks_for(long long n, int threads) { return (int)((n + threads - 1) / threads); }

}  // namespace

// ------------------------------------------------------------------------------ launchers

// The persistent RMSNorm kernels run with a fixed number of 256-thread blocks (a few per SM)
// however many rows there are; ELFB_RMS_PERSISTENT=0 selects the one-block-per-row kernels.
static const bool g_rms_persistent = []() {
  const char* e = getenv("ELFB_RMS_PERSISTENT");
  return !(e && e[0] == '0');
}();
constexpr int RMS_FWD_BLOCKS = 592;  // 4 per SM on 148 SMs (64 registers per thread at dim 4096)
constexpr int RMS_BWD_BLOCKS = 296;  // 2 per SM (128 registers per thread); also the scratch rows the backward writes
static inline int rms_persistent_grid(int rows, int blocks) { return rows < blocks ? (rows > 0 ? rows : 1) : blocks; }

cudaError_t rmsnorm_forward(const void* x, const void* residual, const void* w, void* y, void* h, float* rstd, int rows,
                            int dim, float eps, cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  if (dim % 8) return cudaErrorInvalidValue;
  const int dim8 = dim / 8;
  if (g_rms_persistent && (dim == 2048 || dim == 4096 || dim == 8192)) {
    const int grid = rms_persistent_grid(rows, RMS_FWD_BLOCKS);
    const Bf16x8 *xp = (const Bf16x8*)x, *rp = (const Bf16x8*)residual, *wp = (const Bf16x8*)w;
    Bf16x8 *yp = (Bf16x8*)y, *hp = (Bf16x8*)h;
#define ELFB_RMS_FWD(RES, VPT) rmsnorm_fwd_persistent_kernel<RES, VPT><<<grid, 256, 0, s>>>(xp, rp, wp, yp, hp, rstd, rows, 1.f / dim, eps)
    if (residual) {
      if (dim == 2048) ELFB_RMS_FWD(true, 1); else if (dim == 4096) ELFB_RMS_FWD(true, 2); else ELFB_RMS_FWD(true, 4);
    } else {
      if (dim == 2048) ELFB_RMS_FWD(false, 1); else if (dim == 4096) ELFB_RMS_FWD(false, 2); else ELFB_RMS_FWD(false, 4);
    }
#undef ELFB_RMS_FWD
    return cudaGetLastError();
  }
  const bool narrow = dim8 <= 128 * RMS_MAX_VEC;
  if (residual) {
    if (narrow)
      rmsnorm_fwd_kernel<true, 128><<<rows, 128, 0, s>>>((const Bf16x8*)x, (const Bf16x8*)residual, (const Bf16x8*)w, (Bf16x8*)y, (Bf16x8*)h, rstd, dim8,
                                                         1.f / dim, eps);
    else
      rmsnorm_fwd_kernel<true, 256><<<rows, 256, 0, s>>>((const Bf16x8*)x, (const Bf16x8*)residual, (const Bf16x8*)w, (Bf16x8*)y, (Bf16x8*)h, rstd, dim8,
                                                         1.f / dim, eps);
  } else {
    if (narrow)
      rmsnorm_fwd_kernel<false, 128><<<rows, 128, 0, s>>>((const Bf16x8*)x, nullptr, (const Bf16x8*)w, (Bf16x8*)y, nullptr, rstd, dim8, 1.f / dim, eps);
    else
      rmsnorm_fwd_kernel<false, 256><<<rows, 256, 0, s>>>((const Bf16x8*)x, nullptr, (const Bf16x8*)w, (Bf16x8*)y, nullptr, rstd, dim8, 1.f / dim, eps);
  }
  return cudaGetLastError();
}

// Scratch rows (of `dim` floats) the backward wants: the persistent kernel writes one partial row
// per block.  With fewer rows available (but at least rmsnorm_backward_min_blocks()) the
// one-block-per-row kernels run instead.
int rmsnorm_backward_blocks(int rows) {
  const int g = rms_persistent_grid(rows, RMS_BWD_BLOCKS);
  return g > RMS_DW_SPLITS ? g : RMS_DW_SPLITS;
}
int rmsnorm_backward_min_blocks() { return RMS_DW_SPLITS; }

cudaError_t rmsnorm_backward(const void* dy, const void* x, const void* w, const float* rstd, const void* dres_in, void* dx,
                             float* dw_partial, int scratch_rows, void* dw, bool dw_bf16, bool accumulate_dw, int rows, int dim,
                             cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  if (dim % 8 || dim > 256 * RMS_MAX_VEC * 8 || scratch_rows < RMS_DW_SPLITS) return cudaErrorInvalidValue;
  const int dim8 = dim / 8;
  if (g_rms_persistent && (dim == 2048 || dim == 4096 || dim == 8192) && scratch_rows >= rms_persistent_grid(rows, RMS_BWD_BLOCKS)) {
    const int grid = rms_persistent_grid(rows, RMS_BWD_BLOCKS);
    const Bf16x8 *gp = (const Bf16x8*)dy, *xp = (const Bf16x8*)x, *wp = (const Bf16x8*)w, *rp = (const Bf16x8*)dres_in;
#define ELFB_RMS_BWD(RES, VPT) rmsnorm_bwd_persistent_kernel<RES, VPT><<<grid, 256, 0, s>>>(gp, xp, wp, rstd, rp, (Bf16x8*)dx, dw_partial, rows, 1.f / dim)
    if (dres_in) {
      if (dim == 2048) ELFB_RMS_BWD(true, 1); else if (dim == 4096) ELFB_RMS_BWD(true, 2); else ELFB_RMS_BWD(true, 4);
    } else {
      if (dim == 2048) ELFB_RMS_BWD(false, 1); else if (dim == 4096) ELFB_RMS_BWD(false, 2); else ELFB_RMS_BWD(false, 4);
    }
#undef ELFB_RMS_BWD
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (dw_bf16) {
      if (!accumulate_dw) return cudaErrorInvalidValue;
      colsum_tall_kernel<__nv_bfloat16><<<(dim + 31) / 32, 256, 0, s>>>(dw_partial, (__nv_bfloat16*)dw, grid, dim, true);
    } else {
      colsum_tall_kernel<float><<<(dim + 31) / 32, 256, 0, s>>>(dw_partial, (float*)dw, grid, dim, accumulate_dw);
    }
    return cudaGetLastError();
  }
  const bool narrow = dim8 <= 128 * RMS_MAX_VEC;
  if (dres_in) {
    if (narrow)
      rmsnorm_bwd_dx_kernel<true, 128><<<rows, 128, 0, s>>>((const Bf16x8*)dy, (const Bf16x8*)x, (const Bf16x8*)w, rstd, (const Bf16x8*)dres_in, (Bf16x8*)dx,
                                                            dim8, 1.f / dim);
    else
      rmsnorm_bwd_dx_kernel<true, 256><<<rows, 256, 0, s>>>((const Bf16x8*)dy, (const Bf16x8*)x, (const Bf16x8*)w, rstd, (const Bf16x8*)dres_in, (Bf16x8*)dx,
                                                            dim8, 1.f / dim);
  } else {
    if (narrow)
      rmsnorm_bwd_dx_kernel<false, 128><<<rows, 128, 0, s>>>((const Bf16x8*)dy, (const Bf16x8*)x, (const Bf16x8*)w, rstd, nullptr, (Bf16x8*)dx, dim8, 1.f / dim);
    else
      rmsnorm_bwd_dx_kernel<false, 256><<<rows, 256, 0, s>>>((const Bf16x8*)dy, (const Bf16x8*)x, (const Bf16x8*)w, rstd, nullptr, (Bf16x8*)dx, dim8, 1.f / dim);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const dim3 grid((dim8 + 31) / 32, RMS_DW_SPLITS);
  rmsnorm_bwd_dw_kernel<<<grid, 256, 0, s>>>((const Bf16x8*)dy, (const Bf16x8*)x, rstd, dw_partial, rows, dim8);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (dw_bf16) {
    if (!accumulate_dw) return cudaErrorInvalidValue;  // a bf16 target is a gradient buffer: always added to
    colsum_add_bf16_kernel<<<blocks_for(dim, 256), 256, 0, s>>>(dw_partial, (__nv_bfloat16*)dw, RMS_DW_SPLITS, dim);
  } else {
    colsum_kernel<<<blocks_for(dim, 256), 256, 0, s>>>(dw_partial, (float*)dw, RMS_DW_SPLITS, dim, accumulate_dw);
  }
  return cudaGetLastError();
}

cudaError_t pack_qkv_grad(const void* dq, const void* dk, const void* dv, void* out, int batch, int seq, int hq, int hkv, int head_dim,
                          const long long* q_strides, const long long* k_strides, const long long* v_strides, const float* cos_t,
                          const float* sin_t, cudaStream_t s) {
  if (head_dim % 8) return cudaErrorInvalidValue;
  for (int i = 0; i < 3; ++i)
    if (q_strides[i] % 8 || k_strides[i] % 8 || v_strides[i] % 8) return cudaErrorInvalidValue;
  if (cos_t != nullptr) {
    const int half = head_dim / 2;
    if (half % 8 || sin_t == nullptr) return cudaErrorInvalidValue;
    const long long n = (long long)batch * seq * (hq + 2 * hkv) * (half / 8);
    if (n == 0) return cudaSuccess;
    pack_qkv_grad_rope_kernel<<<blocks_for(n, 256), 256, 0, s>>>((const __nv_bfloat16*)dq, (const __nv_bfloat16*)dk, (const __nv_bfloat16*)dv,
                                                                 (__nv_bfloat16*)out, cos_t, sin_t, n, seq, hq, hkv, half, q_strides[0], q_strides[1],
                                                                 q_strides[2], k_strides[0], k_strides[1], k_strides[2], v_strides[0], v_strides[1],
                                                                 v_strides[2]);
    return cudaGetLastError();
  }
  const int d8 = head_dim / 8;
  const long long total = (long long)batch * seq * (hq + 2 * hkv) * d8;
  if (total == 0) return cudaSuccess;
  pack_qkv_grad_kernel<<<blocks_for(total, 256), 256, 0, s>>>((const Bf16x8*)dq, (const Bf16x8*)dk, (const Bf16x8*)dv, (Bf16x8*)out, total, seq, hq, hkv, d8,
                                                              q_strides[0] / 8, q_strides[1] / 8, q_strides[2] / 8, k_strides[0] / 8, k_strides[1] / 8,
                                                              k_strides[2] / 8, v_strides[0] / 8, v_strides[1] / 8, v_strides[2] / 8);
  return cudaGetLastError();
}

cudaError_t residual_add(void* out, const void* res, long long n, cudaStream_t s) {
  if (n % 8) return cudaErrorInvalidValue;
  if (n == 0) return cudaSuccess;
  residual_add_kernel<<<blocks_for(n / 8, 256), 256, 0, s>>>((Bf16x8*)out, (const Bf16x8*)res, n / 8);
  return cudaGetLastError();
}

cudaError_t rope_inplace(void* x, const float* cos_t, const float* sin_t, int rows, int row_stride, int n_rot_heads,
                         int head_dim, int seq_len, float sign, cudaStream_t s) {
  const int half = head_dim / 2;
  if (half % 8 || row_stride % 8) return cudaErrorInvalidValue;
  const long long total = (long long)rows * n_rot_heads * (half / 8);
  if (total == 0) return cudaSuccess;
  rope_kernel<<<blocks_for(total, 256), 256, 0, s>>>((__nv_bfloat16*)x, cos_t, sin_t, total, row_stride, n_rot_heads, half,
                                                     seq_len, sign);
  return cudaGetLastError();
}

cudaError_t swiglu_forward(const void* gu, void* out, int rows, int f, cudaStream_t s) {
  if (f % 8) return cudaErrorInvalidValue;
  const long long total = (long long)rows * (f / 8);
  if (total == 0) return cudaSuccess;
  swiglu_fwd_kernel<<<blocks_for(total, 256), 256, 0, s>>>((const Bf16x8*)gu, (Bf16x8*)out, total, f / 8);
  return cudaGetLastError();
}
cudaError_t swiglu_backward(const void* dout, const void* gu, void* dgu, int rows, int f, cudaStream_t s) {
  if (f % 8) return cudaErrorInvalidValue;
  const long long total = (long long)rows * (f / 8);
  if (total == 0) return cudaSuccess;
  swiglu_bwd_kernel<<<blocks_for(total, 256), 256, 0, s>>>((const Bf16x8*)dout, (const Bf16x8*)gu, (Bf16x8*)dgu, total, f / 8);
  return cudaGetLastError();
}

cudaError_t cross_entropy_forward(const void* logits, const int64_t* targets, float* loss, float* lse, int rows, int vocab,
                                  long long ld, int64_t ignore_index, cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  if (ld % 8) return cudaErrorInvalidValue;
  ce_fwd_kernel<<<rows, CE_THREADS, 0, s>>>((const __nv_bfloat16*)logits, targets, loss, lse, vocab, ld, ignore_index);
  return cudaGetLastError();
}
cudaError_t cross_entropy_backward(const void* logits, void* dlogits, const int64_t* targets, const float* lse,
                                   const float* gscale, float scale, int rows, int vocab, long long ld, int64_t ignore_index,
                                   cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  if (ld % 8) return cudaErrorInvalidValue;
  ce_bwd_kernel<<<rows, CE_THREADS, 0, s>>>((const __nv_bfloat16*)logits, (__nv_bfloat16*)dlogits, targets, lse, gscale, scale,
                                            vocab, ld, ignore_index);
  return cudaGetLastError();
}

cudaError_t cross_entropy_chunk_stats(const void* logits, const int64_t* targets, float* run_max, float* run_sum, float* tgt_logit, int rows,
                                      int width, long long ld, long long col0, bool first, cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  if (ld % 8) return cudaErrorInvalidValue;
  ce_chunk_stats_kernel<<<rows, CE_THREADS, 0, s>>>((const __nv_bfloat16*)logits, targets, run_max, run_sum, tgt_logit, width, ld, col0, first);
  return cudaGetLastError();
}
cudaError_t cross_entropy_chunk_grad(void* logits, const int64_t* targets, const float* lse, const float* gscale, float scale, int rows, int width,
                                     long long ld, long long col0, long long vocab, int64_t ignore_index, cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  if (ld % 8) return cudaErrorInvalidValue;
  ce_chunk_grad_kernel<<<rows, CE_THREADS, 0, s>>>((__nv_bfloat16*)logits, targets, lse, gscale, scale, width, ld, col0, vocab, ignore_index);
  return cudaGetLastError();
}

cudaError_t embedding_forward(const void* table, const int64_t* ids, void* out, int rows, int dim, long long vocab, int* status,
                              cudaStream_t s) {
  if (dim % 8) return cudaErrorInvalidValue;
  const long long total = (long long)rows * (dim / 8);
  if (total == 0) return cudaSuccess;
  embedding_fwd_kernel<<<blocks_for(total, 256), 256, 0, s>>>((const Bf16x8*)table, ids, (Bf16x8*)out, total, dim / 8, vocab, status);
  return cudaGetLastError();
}
cudaError_t embedding_backward(const void* dout, const int64_t* ids, void* dtable, bool dtable_f32, int rows, int dim, long long vocab,
                               int* status, cudaStream_t s) {
  if (dim % 2) return cudaErrorInvalidValue;
  const long long total = (long long)rows * (dim / 2);
  if (total == 0) return cudaSuccess;
  if (dtable_f32)
    embedding_bwd_kernel<true><<<blocks_for(total, 256), 256, 0, s>>>((const __nv_bfloat162*)dout, ids, dtable, total, dim / 2, vocab, status);
  else
    embedding_bwd_kernel<false><<<blocks_for(total, 256), 256, 0, s>>>((const __nv_bfloat162*)dout, ids, dtable, total, dim / 2, vocab, status);
  return cudaGetLastError();
}

cudaError_t embedding_backward_sorted(const void* dout, const int64_t* sorted_ids, const int64_t* perm, void* grad, bool grad_f32, int rows,
                                      int dim, long long vocab, cudaStream_t s) {
  if (dim % 8) return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  if (grad_f32)
    embedding_bwd_sorted_kernel<true><<<rows, 256, 0, s>>>((const Bf16x8*)dout, sorted_ids, perm, grad, rows, dim / 8, vocab);
  else
    embedding_bwd_sorted_kernel<false><<<rows, 256, 0, s>>>((const Bf16x8*)dout, sorted_ids, perm, grad, rows, dim / 8, vocab);
  return cudaGetLastError();
}

cudaError_t adamw_step(void* p_bf16, const void* grad, bool grad_f32, float* master, float* m, float* v, long long n,
                       float lr, float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2,
                       float grad_scale, const int* status, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  const long long n8 = (n + 7) / 8;
  const float decay = 1.f - lr * weight_decay;
  if (grad_f32)
    adamw_kernel<true><<<blocks_for(n8, 256), 256, 0, s>>>((Bf16x8*)p_bf16, grad, master, m, v, n8, n, lr, beta1, beta2, eps,
                                                           decay, 1.f / bc1, 1.f / bc2, grad_scale, status);
  else
    adamw_kernel<false><<<blocks_for(n8, 256), 256, 0, s>>>((Bf16x8*)p_bf16, grad, master, m, v, n8, n, lr, beta1, beta2, eps,
                                                            decay, 1.f / bc1, 1.f / bc2, grad_scale, status);
  return cudaGetLastError();
}

cudaError_t scale_bf16(void* x, long long n, float a, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  const long long n8 = (n + 7) / 8;
  scale_bf16_kernel<<<blocks_for(n8, 256), 256, 0, s>>>((Bf16x8*)x, n8, n, a);
  return cudaGetLastError();
}

}  // namespace elfb
