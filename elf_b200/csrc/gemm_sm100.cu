// Persistent warp-specialised tcgen05 GEMM for sm_100a.
//
//   D[M,N] (+)= A . B (+ bias[N])        bf16/fp16 operands, fp32 accumulation in TMEM
//
// The three linear-layer GEMMs differ only in which operand dimension is contiguous:
//   forward      Y  = X . W^T    A = X  [M,K]  K-major    B = W  [N,K]  K-major
//   input grad   dX = dY . W     A = dY [M,K]  K-major    B = W  [K,N]  MN-major
//   weight grad  dW = dY^T . X   A = dY [K,M]  MN-major   B = X  [K,N]  MN-major
// (K always names the reduction dimension of the product at hand.)
//
// Structure per CTA (192 threads, one CTA per SM, grid = min(#tiles, #SMs)):
//   warp 0      TMA producer: fills a 4-stage ring of (A 128x64, B 256x64) bf16 tiles,
//               128B-swizzled, completion on `full[s]`.
//   warp 1      MMA issuer: one thread issues 128x256x16 tcgen05.mma into one of two TMEM
//               accumulators (2 x 256 columns = all 512 columns), releasing ring slots with
//               tcgen05.commit -> `empty[s]` and finished tiles with commit -> `acc_full[a]`.
//   warps 2..5  epilogue: tcgen05.ld the accumulator (thread = row, 32 columns at a time),
//               add bias / the previous contents of D, convert, store; then `acc_empty[a]`.
// While the epilogue drains accumulator a, the mainloop of the next tile fills 1-a.
//
// Every mbarrier wait is bounded (see sm100_ptx.cuh); on a timeout the CTA raises a shared
// abort flag, all roles fall through to the common exit, TMEM is released and an error
// code is written to `status`.

#include <cstdio>

#include "sm100_ptx.cuh"
#include "gemm_epilogue.cuh"
#include "dp_signal.cuh"
#include "gemm_sm100.h"

namespace elfb {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 8;  // rasterisation: tiles of GROUP_M consecutive M-blocks share B panels in L2
constexpr size_t SMEM_BYTES = size_t(STAGES) * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;

// A work unit is a 128-row slab of BN/split columns.  Units [0, full_units) are whole
// 128x256 tiles of the complete waves; the tiles of the last, partial wave are cut into
// `split` column strips each (split = 1, 2 or 4) so that the tail keeps all SMs busy for a
// fraction of a tile time instead of leaving most of them idle for a whole one.
struct WorkUnit {
  int m, n0, width;
};

struct Schedule {
  int tiles_m, tiles_n, full_tiles, split, total_units;
};

__host__ __device__ inline Schedule make_schedule(int M, int N, int num_ctas, int max_split) {
  Schedule s;
  s.tiles_m = (M + BM - 1) / BM;
  s.tiles_n = (N + BN - 1) / BN;
  const int tiles = s.tiles_m * s.tiles_n;
  const int rem = tiles % num_ctas;
  s.split = 1;
  if (rem != 0 && tiles > rem) {  // only behind at least one complete wave
    // cost of the tail in tile times: ceil(rem * f / P) / f
    int best_num = 1, best_den = 1;  // f = 1: one more wave
    for (int f = 2; f <= max_split; f *= 2) {
      const int waves = (rem * f + num_ctas - 1) / num_ctas;
      if (waves * best_den < best_num * f) {
        best_num = waves;
        best_den = f;
        s.split = f;
      }
    }
  }
  s.full_tiles = s.split == 1 ? tiles : tiles - rem;
  s.total_units = s.full_tiles + (tiles - s.full_tiles) * s.split;
  return s;
}

__device__ __forceinline__ WorkUnit work_unit(int unit, const Schedule& s) {
  int tile = unit, strip = 0, width = BN;
  if (unit >= s.full_tiles) {
    const int u = unit - s.full_tiles;
    tile = s.full_tiles + u / s.split;
    strip = u % s.split;
    width = BN / s.split;
  }
  const int per_group = GROUP_M * s.tiles_n;
  const int group = tile / per_group;
  const int first_m = group * GROUP_M;
  const int rows = min(GROUP_M, s.tiles_m - first_m);
  const int in_group = tile - group * per_group;
  return {first_m + in_group % rows, (in_group / rows) * BN + strip * width, width};
}

template <bool A_MN, bool B_MN, bool OUT_F32, bool ACCUM, bool BIAS>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_b_half, const __grid_constant__ CUtensorMap tmap_b_quarter,
                    void* __restrict__ d_ptr, const void* __restrict__ bias_ptr, int M, int N, int K, long long ldd,
                    uint32_t fmt, float alpha, int max_split, int* __restrict__ status, const __grid_constant__ PushTarget push) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_aligned + size_t(STAGES) * STAGE_BYTES);
  // barrier slots: full[0..S), empty[S..2S), acc_full[2S..2S+2), acc_empty[2S+2..2S+4)
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
  auto acc_empty_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const Schedule sched = make_schedule(M, N, gridDim.x, max_split);
  const int num_units = sched.total_units;
  const int k_blocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 4);  // one arrival per epilogue warp
    }
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
        const WorkUnit wu = work_unit(unit, sched);
        const int m0 = wu.m * BM, n0 = wu.n0;
        const uint32_t stage_tx = A_BYTES + wu.width * BK * 2;
        const CUtensorMap* tb_k = wu.width == BN ? &tmap_b : (wu.width == BN / 2 ? &tmap_b_half : &tmap_b_quarter);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          const uint32_t bar = full_bar(stage);
          mbar_arrive_expect_tx(bar, stage_tx);
          const int k0 = kb * BK;
          if (A_MN) {
            // global [K rows][M contiguous]: one 64(M) x 64(K) box per 64 rows of the tile
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * (BK * 128), &tmap_a, bar, m0 + 64 * j, k0);
          } else {
            tma_load_2d(sa, &tmap_a, bar, k0, m0);  // global [M rows][K contiguous]: 64(K) x 128(M)
          }
          if (B_MN) {
            for (int j = 0; j < wu.width / 64; ++j) tma_load_2d(sb + j * (BK * 128), &tmap_b, bar, n0 + 64 * j, k0);
          } else {
            tma_load_2d(sb, tb_k, bar, k0, n0);  // 64(K) x width(N)
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_full = make_idesc_f16(fmt, BM, BN, A_MN ? 1u : 0u, B_MN ? 1u : 0u);
      // K-major: 64-element (128 B) rows, 8-row groups 1024 B apart; a k-step of 16 = 32 B.
      // MN-major: 64-wide boxes of BK rows; 8-row k-groups 1024 B apart; k-step of 16 rows = 2048 B.
      constexpr uint32_t A_LBO = A_MN ? BK * 128 : 0, B_LBO = B_MN ? BK * 128 : 0;
      constexpr uint32_t A_KSTEP = A_MN ? UMMA_K * 128 : UMMA_K * 2, B_KSTEP = B_MN ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
        const int width = unit >= sched.full_tiles ? BN / sched.split : BN;
        const uint32_t idesc = width == BN ? idesc_full : make_idesc_f16(fmt, BM, width, A_MN ? 1u : 0u, B_MN ? 1u : 0u);
        if (!mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u, abort_flag)) break;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = make_smem_desc_sw128(sa + k * A_KSTEP, A_LBO, 1024);
            const uint64_t db = make_smem_desc_sw128(sb + k * B_KSTEP, B_LBO, 1024);
            umma_ss(tmem_d, da, db, idesc, (kb | k) ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));  // slot reusable once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(acc_full_bar(acc));  // accumulator complete
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int unit = blockIdx.x; unit < num_units; unit += gridDim.x) {
      const WorkUnit wu = work_unit(unit, sched);
      const int row = wu.m * BM + quarter * 32 + lane;
      const int n0 = wu.n0;
      if (!mbar_wait(acc_full_bar(acc), acc_phase, abort_flag)) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < wu.width / 32; ++c) {
        const int col = n0 + c * 32;
        if (col >= N) break;  // warp-uniform
        uint32_t v[32];
        tmem_ld_32x32b_x32(taddr + c * 32, v);
        tmem_ld_wait();
        store_accumulator_chunk<OUT_F32, ACCUM, BIAS>(v, row, col, M, N, d_ptr, ldd, bias_ptr, fmt, alpha, push);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(acc));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  }

  // ------------------------------------------------------------------ common exit
  if (push.n_peers > 0) signal_peers_when_last(push.done_counter, push.peer_flag, push.n_peers, push.flag_value);
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) {
      // let TMA copies that are still in flight land before the CTA's shared memory goes away
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) {
      }
      if (status != nullptr && atomicCAS(status, kOk, kErrBarrierTimeout) == kOk) {
        status[1] = blockIdx.x;
        status[2] = M;
        status[3] = N;
      }
    }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ----------------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------------

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn get_encode_fn() {
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || p == nullptr) return nullptr;
    fn = reinterpret_cast<EncodeFn>(p);
  }
  return fn;
}

// 2D row-major 16-bit matrix [rows][cols] with leading dimension `ld` elements;
// box = (box_cols inner, box_rows outer), 128B swizzle, zero fill outside the matrix.
const char* make_tmap_2d(CUtensorMap* out, const void* ptr, int fmt, uint64_t rows, uint64_t cols, uint64_t ld,
                         uint32_t box_cols, uint32_t box_rows) {
  // Driver entry points need a CUDA context current on the calling thread; autograd runs
  // backward passes on worker threads that may not have made a runtime call yet.
  static thread_local bool context_ready = false;
  if (!context_ready) {
    cudaFree(nullptr);
    context_ready = true;
  }
  EncodeFn enc = get_encode_fn();
  if (!enc) return "cuTensorMapEncodeTiled entry point not found";
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0) return "TMA operand base address is not 16-byte aligned";
  if ((ld * 2) % 16 != 0) return "TMA operand row pitch is not a multiple of 16 bytes";
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                   const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS) return nullptr;
  static thread_local char msg[256];
  snprintf(msg, sizeof(msg), "cuTensorMapEncodeTiled failed (CUresult %d) for ptr=%p rows=%llu cols=%llu ld=%llu box=(%u,%u)", (int)r, ptr,
           (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld, box_cols, box_rows);
  return msg;
}

// Row-major [rows][cols] output matrix of 16-bit (fmt 0/1) or fp32 (fmt 2) elements for TMA
// stores / add-reductions: 128-byte swizzled boxes of box_cols x box_rows.
const char* make_tmap_out(CUtensorMap* out, const void* ptr, int fmt, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                          uint32_t box_rows) {
  EncodeFn enc = get_encode_fn();
  if (!enc) return "cuTensorMapEncodeTiled entry point not found";
  const uint64_t esz = fmt == 2 ? 4 : 2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * esz};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = fmt == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : (fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  CUresult r = enc(out, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? nullptr : "cuTensorMapEncodeTiled failed for the output matrix";
}

template <bool A_MN, bool B_MN, bool OUT_F32, bool ACCUM, bool BIAS>
static cudaError_t launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const CUtensorMap& tb4, void* d, const void* bias, int M, int N, int K,
                              long long ldd, uint32_t fmt, float alpha, int max_split, int* status, const PushTarget& push, int num_sms, cudaStream_t stream) {
  auto kern = gemm_tcgen05_kernel<A_MN, B_MN, OUT_F32, ACCUM, BIAS>;
  // function attributes are per device: remember which devices of this process have been set up
  static bool configured[kMaxDevices] = {};
  int dev = 0;
  if (cudaError_t e = cudaGetDevice(&dev); e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < kMaxDevices) configured[dev] = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  kern<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, tb2, tb4, d, bias, M, N, K, ldd, fmt, alpha, max_split, status, push);
  flush_bounds_record(status, stream);
  return cudaGetLastError();
}

template <bool A_MN, bool B_MN>
static cudaError_t dispatch_epilogue(const GemmArgs& g, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const CUtensorMap& tb4,
                                     int num_sms, cudaStream_t s) {
#define ELFB_LAUNCH(F32, ACC, BI) \
  return launch_one<A_MN, B_MN, F32, ACC, BI>(ta, tb, tb2, tb4, g.d, g.bias, g.M, g.N, g.K, g.ldd, (uint32_t)g.fmt, g.alpha, g.split_tail ? 4 : 1, g.status, g.push, num_sms, s)
  if (g.out_f32) {
    if (g.accumulate) { if (g.bias) ELFB_LAUNCH(true, true, true); else ELFB_LAUNCH(true, true, false); }
    else              { if (g.bias) ELFB_LAUNCH(true, false, true); else ELFB_LAUNCH(true, false, false); }
  } else {
    if (g.accumulate) { if (g.bias) ELFB_LAUNCH(false, true, true); else ELFB_LAUNCH(false, true, false); }
    else              { if (g.bias) ELFB_LAUNCH(false, false, true); else ELFB_LAUNCH(false, false, false); }
  }
#undef ELFB_LAUNCH
}

const char* gemm_tcgen05(const GemmArgs& g, int num_sms, cudaStream_t stream) {
  if (g.M <= 0 || g.N <= 0 || g.K <= 0) return nullptr;
  if (g.variant == 1 && num_sms >= 2) return gemm_tcgen05_pair(g, num_sms, stream);
  CUtensorMap ta, tb, tb2, tb4;
  const char* err;
  if (g.a_mn_major) err = make_tmap_2d(&ta, g.a, g.fmt, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)g.lda, 64, BK);
  else              err = make_tmap_2d(&ta, g.a, g.fmt, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.lda, BK, BM);
  if (err) return err;
  if (g.b_mn_major) err = make_tmap_2d(&tb, g.b, g.fmt, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.ldb, 64, BK);
  else              err = make_tmap_2d(&tb, g.b, g.fmt, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb, BK, BN);
  if (err) return err;
  // K-major B strips of the split tail wave need their own box heights; MN-major B is
  // fetched in 64-wide boxes whatever the strip width
  tb2 = tb;
  tb4 = tb;
  if (!g.b_mn_major) {
    err = make_tmap_2d(&tb2, g.b, g.fmt, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb, BK, BN / 2);
    if (err) return err;
    err = make_tmap_2d(&tb4, g.b, g.fmt, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb, BK, BN / 4);
    if (err) return err;
  }
  const int esz = g.out_f32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(g.d) & 15) != 0 || (g.ldd * esz) % 16 != 0) return "GEMM output must be 16-byte aligned with a 16-byte multiple row pitch";
  cudaError_t e;
  if (g.a_mn_major && g.b_mn_major) e = dispatch_epilogue<true, true>(g, ta, tb, tb2, tb4, num_sms, stream);
  else if (!g.a_mn_major && g.b_mn_major) e = dispatch_epilogue<false, true>(g, ta, tb, tb2, tb4, num_sms, stream);
  else if (!g.a_mn_major && !g.b_mn_major) e = dispatch_epilogue<false, false>(g, ta, tb, tb2, tb4, num_sms, stream);
  else e = dispatch_epilogue<true, false>(g, ta, tb, tb2, tb4, num_sms, stream);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

#ifdef ELF_BOUNDS_CHECK
namespace {
// Issues a store and a reduce whose coordinates break the rules (odd x; negative y).  The checked
// wrappers record the first one and skip both, so nothing reaches the hardware: the tensor map
// pointer is never used.
__global__ void bounds_selftest_kernel() {
  tma_store_2d(nullptr, 0u, 3, 0);
  tma_reduce_add_2d(nullptr, 0u, 8, -4);
}
}  // namespace

bool bounds_check_build() { return true; }
cudaError_t bounds_check_selftest(int* status, cudaStream_t stream) {
  bounds_selftest_kernel<<<1, 1, 0, stream>>>();
  flush_bounds_record(status, stream);
  return cudaGetLastError();
}
#else
bool bounds_check_build() { return false; }
cudaError_t bounds_check_selftest(int*, cudaStream_t) { return cudaErrorNotSupported; }
#endif

}  // namespace elfb
