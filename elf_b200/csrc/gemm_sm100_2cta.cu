// CTA-pair variant of the tcgen05 GEMM: two CTAs on neighbouring SMs (a cluster of 2) share
// one 256x256 output tile through `tcgen05.mma.cta_group::2`.
//
// Each CTA owns 128 of the tile's 256 rows: it TMA-loads its own A slab (128 x 64) and HALF
// of the B slab (128 of the 256 B rows) into its own shared memory and receives its 128
// accumulator rows in its own TMEM.  Per flop, each SM therefore reads half as much B from
// shared memory as in the single-CTA kernel (and fetches half as much from L2), which is
// what lets the tensor pipe run closer to its peak under the power cap.
//
// Synchronisation (every wait bounded, see sm100_ptx.cuh):
//   full[s]      lives in the EVEN CTA (the leader).  The leader's producer arms it with the
//                byte count of both CTAs' loads; both CTAs' TMA copies complete on it
//                (the odd CTA addresses it through the cluster window; no multicast).
//   empty[s]     one per CTA; the leader's MMA thread commits to both after the MMAs that
//                read stage s.
//   acc_full[a]  one per CTA; committed by the leader after the last MMA of a tile.
//   acc_empty[a] in the leader; the epilogue warps of both CTAs arrive on it (8 arrivals).
// Only the leader's MMA thread issues MMAs.  TMEM is allocated and freed with the
// cta_group::2 forms by warp 1 of both CTAs.

#include <cstdio>
#include <cstdlib>

#include "sm100_ptx.cuh"
#include "gemm_epilogue.cuh"
#include "dp_signal.cuh"
#include "gemm_sm100.h"

namespace elfb {

namespace pair {

constexpr int BM = 128;          // rows per CTA (256 per pair)
constexpr int BN = 256;          // columns per pair tile
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;        // 16 KiB
constexpr int B_BYTES = (BN / 2) * BK * 2;  // 16 KiB: this CTA's half of the B slab
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int DEFAULT_GROUP_M = 4;  // tile rows (of 256) that are swept together before moving to the next columns
constexpr int STAGING_BYTES = 2 * 16384;  // two 128-row x 128-byte chunks for the TMA-store epilogue
constexpr size_t SMEM_BYTES = size_t(STAGES) * STAGE_BYTES + STAGING_BYTES + 1024 + 256;

// Tensor maps over the peers' copies of D (same shape and pitch as the local D), used when the
// epilogue also pushes its tiles to other GPUs.
struct alignas(64) PeerMaps {
  CUtensorMap m[kMaxPeers];
};

struct WorkUnit {
  int m, n0;      // tile row (in 256-row units) and first output column
  int kb0, kb1;   // range of 64-wide k-blocks this unit contracts over
  int part;       // index of this unit among the k-parts of its tile (0 when the tile is whole)
  bool partial;   // true: the unit holds a partial sum and must add it to D
};
// Tiles are dealt round-robin to the CTA pairs.  When the tile count is not a multiple of
// the pair count the last, partly filled wave would cost a whole tile time with most SMs
// idle; instead each tile of that wave is split along K into `ksplit` units that run on
// different pairs and add their partial sums to D (TMA add-reduce in L2).  Unlike a split
// along N this keeps the 256x256 tile's ratio of MMA work to bytes loaded.
struct Schedule {
  int tiles_m, tiles_n, full_tiles, ksplit, total_units, group_m;
};

__host__ __device__ inline Schedule make_schedule(int M, int N, int k_blocks, int num_pairs, int max_split, int group_m) {
  Schedule s;
  s.group_m = group_m;
  s.tiles_m = (M + 2 * BM - 1) / (2 * BM);
  s.tiles_n = (N + BN - 1) / BN;
  const int tiles = s.tiles_m * s.tiles_n;
  const int rem = tiles % num_pairs;
  s.ksplit = 1;
  if (rem != 0 && tiles > rem) {
    // cost of the last wave in 1/840 tile times, plus a charge per extra part for its exposed epilogue
    int best = 840;
    for (int f = 2; f <= max_split && f * 4 <= k_blocks; ++f) {
      const int waves = (rem * f + num_pairs - 1) / num_pairs;
      const int cost = waves * 840 / f + 30 * (f - 1);
      if (cost < best) {
        best = cost;
        s.ksplit = f;
      }
    }
  }
  s.full_tiles = s.ksplit == 1 ? tiles : tiles - rem;
  s.total_units = s.full_tiles + (tiles - s.full_tiles) * s.ksplit;
  return s;
}

__host__ __device__ inline void tile_coords(int tile, const Schedule& s, int* m, int* n) {
  const int per_group = s.group_m * s.tiles_n;
  const int group = tile / per_group;
  const int first_m = group * s.group_m;
  const int rows = (s.tiles_m - first_m) < s.group_m ? (s.tiles_m - first_m) : s.group_m;
  const int in_group = tile - group * per_group;
  *m = first_m + in_group % rows;
  *n = in_group / rows;
}

__device__ __forceinline__ WorkUnit work_unit(int unit, const Schedule& s, int k_blocks) {
  WorkUnit wu;
  int tile = unit;
  wu.kb0 = 0;
  wu.kb1 = k_blocks;
  wu.part = 0;
  wu.partial = false;
  if (unit >= s.full_tiles) {
    // parts of one tile are `rem` units apart, so they land on different pairs
    const int rem = (s.total_units - s.full_tiles) / s.ksplit;
    const int u = unit - s.full_tiles;
    tile = s.full_tiles + u % rem;
    wu.part = u / rem;
    wu.kb0 = int((long long)k_blocks * wu.part / s.ksplit);
    wu.kb1 = int((long long)k_blocks * (wu.part + 1) / s.ksplit);
    wu.partial = true;
  }
  int n;
  tile_coords(tile, s, &wu.m, &n);
  wu.n0 = n * BN;
  return wu;
}

template <bool A_MN, bool B_MN, bool OUT_F32, bool ACCUM, bool BIAS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ CUtensorMap tmap_d, void* __restrict__ d_ptr, const void* __restrict__ bias_ptr, int M, int N, int K, long long ldd,
                         uint32_t fmt, float alpha, int max_split, int group_m, int* __restrict__ status, const __grid_constant__ PushTarget push,
                         const __grid_constant__ PeerMaps peer_maps) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t staging_base = smem_base + STAGES * STAGE_BYTES;  // 1024-byte aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_aligned + size_t(STAGES) * STAGE_BYTES + STAGING_BYTES);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
  auto acc_empty_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = leader, 1 = peer
  const bool leader = cta == 0;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int k_blocks = (K + BK - 1) / BK;
  const Schedule sched = make_schedule(M, N, k_blocks, num_pairs, max_split, group_m);
  const int num_units = sched.total_units;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);   // used in the leader only: its producer's arrive.expect_tx
      mbar_init(empty_bar(s), 1);  // one commit per use
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 8);  // used in the leader only: 4 epilogue warps of each CTA
    }
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before anyone touches the peer's
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = pair_id; unit < num_units && ok; unit += num_pairs) {
        const WorkUnit wu = work_unit(unit, sched, k_blocks);
        const int m0 = wu.m * (2 * BM) + int(cta) * BM;  // this CTA's 128 rows
        constexpr int half = BN / 2;
        const int n0 = wu.n0 + int(cta) * half;          // this CTA's half of the B rows
        constexpr uint32_t pair_tx = 2u * (A_BYTES + B_BYTES);
        for (int kb = wu.kb0; kb < wu.kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          const uint32_t bar = map_to_cta(full_bar(stage), 0);  // the leader's barrier
          if (leader) mbar_arrive_expect_tx(full_bar(stage), pair_tx);
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * (BK * 128), &tmap_a, bar, m0 + 64 * j, k0);
          } else {
            tma_load_2d_pair(sa, &tmap_a, bar, k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < half / 64; ++j) tma_load_2d_pair(sb + j * (BK * 128), &tmap_b, bar, n0 + 64 * j, k0);
          } else {
            tma_load_2d_pair(sb, &tmap_b, bar, k0, n0);
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
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (leader && lane == 0) {
      constexpr uint32_t A_LBO = A_MN ? BK * 128 : 0, B_LBO = B_MN ? BK * 128 : 0;
      constexpr uint32_t A_KSTEP = A_MN ? UMMA_K * 128 : UMMA_K * 2, B_KSTEP = B_MN ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      const uint32_t idesc = make_idesc_f16(fmt, 2 * BM, BN, A_MN ? 1u : 0u, B_MN ? 1u : 0u);
      for (int unit = pair_id; unit < num_units && ok; unit += num_pairs) {
        const WorkUnit wu = work_unit(unit, sched, k_blocks);
        if (!mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u, abort_flag)) break;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = wu.kb0; kb < wu.kb1; ++kb) {
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
            umma_ss_pair(tmem_d, da, db, idesc, (kb > wu.kb0 || k) ? 1u : 0u);
          }
          umma_commit_pair(map_to_cta(empty_bar(stage), 0));
          umma_commit_pair(map_to_cta(empty_bar(stage), 1));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit_pair(map_to_cta(acc_full_bar(acc), 0));
        umma_commit_pair(map_to_cta(acc_full_bar(acc), 1));
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    // The tile leaves through shared memory: each thread converts its row of a 128-byte-wide
    // column chunk into a swizzled staging buffer and one thread hands the chunk to TMA (store,
    // or add-reduce in L2 when accumulating), so the LSU issues no global stores and D is
    // written in full lines.  With a push target (once per step and matrix) the same staged
    // chunk is also TMA-stored into every peer's copy of D over NVLink; when that launch
    // accumulates, the threads read the old values of their rows themselves and the finished
    // sum is stored (locally and remotely) instead of being add-reduced.
    const int quarter = warp & 3;
    const int ep_tid = threadIdx.x - 64;  // 0..127 over the four epilogue warps
    int acc = 0;
    uint32_t acc_phase = 0;
    const uint32_t leader_acc_empty[2] = {map_to_cta(acc_empty_bar(0), 0), map_to_cta(acc_empty_bar(1), 0)};
    const bool pushing = push.n_peers > 0;
    constexpr int CHUNK_COLS = OUT_F32 ? 32 : 64;  // 128 bytes of output per row
    int chunk_counter = 0;
    for (int unit = pair_id; unit < num_units; unit += num_pairs) {
      const WorkUnit wu = work_unit(unit, sched, k_blocks);
      const int row0 = wu.m * (2 * BM) + int(cta) * BM;
      const int row = row0 + quarter * 32 + lane;
      const bool add_bias = BIAS && wu.part == 0;
      const int n0 = wu.n0;
      if (!mbar_wait(acc_full_bar(acc), acc_phase, abort_flag)) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
      {
        const int r_local = quarter * 32 + lane;          // row inside this CTA's 128-row slab
        const uint32_t swz = uint32_t(r_local & 7);
#pragma unroll 1
        for (int c = 0; c < BN / CHUNK_COLS; ++c) {
          const int col = n0 + c * CHUNK_COLS;
          if (col >= N) break;
          const uint32_t buf = staging_base + uint32_t(chunk_counter & 1) * 16384u;
          // the chunk that used this buffer two chunks ago must have been read out by TMA
          if (ep_tid == 0) tma_store_wait_read<1>();
          named_barrier_sync(1, 128);
          const uint32_t row_base = buf + uint32_t(r_local) * 128u;
#pragma unroll
          for (int h = 0; h < CHUNK_COLS / 32; ++h) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(taddr + c * CHUNK_COLS + h * 32, v);
            tmem_ld_wait();
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]) * alpha;
            if (add_bias) {
              if (OUT_F32) {
                const float* b = reinterpret_cast<const float*>(bias_ptr) + col + h * 32;
#pragma unroll
                for (int j = 0; j < 32; ++j) f[j] += (col + h * 32 + j < N) ? b[j] : 0.f;
              } else {
                const uint16_t* b = reinterpret_cast<const uint16_t*>(bias_ptr) + col + h * 32;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  const uint16_t hb = (col + h * 32 + j < N) ? b[j] : uint16_t(0);
                  f[j] += fmt == 1u ? __bfloat162float(__ushort_as_bfloat16(hb)) : __half2float(__ushort_as_half(hb));
                }
              }
            }
            if (ACCUM && pushing && row < M) {  // the sum itself is stored: fetch what D holds
              const int c0 = col + h * 32;
              if (OUT_F32) {
                const float* old = reinterpret_cast<const float*>(d_ptr) + (long long)row * ldd + c0;
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                  if (c0 + 4 * q + 4 <= N) {
                    const float4 o4 = *reinterpret_cast<const float4*>(old + 4 * q);
                    f[4 * q] += o4.x; f[4 * q + 1] += o4.y; f[4 * q + 2] += o4.z; f[4 * q + 3] += o4.w;
                  } else {
#pragma unroll
                    for (int t = 0; t < 4; ++t)
                      if (c0 + 4 * q + t < N) f[4 * q + t] += old[4 * q + t];
                  }
                }
              } else {
                const uint16_t* old = reinterpret_cast<const uint16_t*>(d_ptr) + (long long)row * ldd + c0;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  if (c0 + 8 * q + 8 <= N) {
                    const uint4 o4 = *reinterpret_cast<const uint4*>(old + 8 * q);
                    const uint32_t w[4] = {o4.x, o4.y, o4.z, o4.w};
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                      const uint16_t lo = uint16_t(w[t] & 0xffffu), hi = uint16_t(w[t] >> 16);
                      f[8 * q + 2 * t] += fmt == 1u ? __bfloat162float(__ushort_as_bfloat16(lo)) : __half2float(__ushort_as_half(lo));
                      f[8 * q + 2 * t + 1] += fmt == 1u ? __bfloat162float(__ushort_as_bfloat16(hi)) : __half2float(__ushort_as_half(hi));
                    }
                  } else {
#pragma unroll
                    for (int t = 0; t < 8; ++t)
                      if (c0 + 8 * q + t < N) f[8 * q + t] += fmt == 1u ? __bfloat162float(__ushort_as_bfloat16(old[8 * q + t])) : __half2float(__ushort_as_half(old[8 * q + t]));
                  }
                }
              }
            }
            if (OUT_F32) {
#pragma unroll
              for (int q = 0; q < 8; ++q) {  // eight 16-byte vectors = the whole 128-byte row
                const uint32_t dst = row_base + ((uint32_t(q) ^ swz) << 4);
                asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "f"(f[4 * q]), "f"(f[4 * q + 1]), "f"(f[4 * q + 2]), "f"(f[4 * q + 3]) : "memory");
              }
            } else {
#pragma unroll
              for (int q = 0; q < 4; ++q) {  // four 16-byte vectors = this half of the row
                uint32_t p0, p1, p2, p3;
                if (fmt == 1u) {
                  p0 = pack_bf16x2(f[8 * q], f[8 * q + 1]); p1 = pack_bf16x2(f[8 * q + 2], f[8 * q + 3]);
                  p2 = pack_bf16x2(f[8 * q + 4], f[8 * q + 5]); p3 = pack_bf16x2(f[8 * q + 6], f[8 * q + 7]);
                } else {
                  p0 = pack_f16x2(f[8 * q], f[8 * q + 1]); p1 = pack_f16x2(f[8 * q + 2], f[8 * q + 3]);
                  p2 = pack_f16x2(f[8 * q + 4], f[8 * q + 5]); p3 = pack_f16x2(f[8 * q + 6], f[8 * q + 7]);
                }
                const uint32_t dst = row_base + ((uint32_t(h * 4 + q) ^ swz) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(p0), "r"(p1), "r"(p2), "r"(p3) : "memory");
              }
            }
          }
          fence_proxy_async_smem();
          named_barrier_sync(1, 128);
          if (ep_tid == 0) {
            if ((ACCUM && !pushing) || wu.partial) tma_reduce_add_2d(&tmap_d, buf, col, row0);
            else tma_store_2d(&tmap_d, buf, col, row0);
            for (int p = 0; p < push.n_peers; ++p) tma_store_2d(&peer_maps.m[p], buf, col, row0);
            tma_store_commit();
          }
          ++chunk_counter;
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_acc_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (ep_tid == 0) tma_store_wait_all();  // every store of this CTA has been performed, the remote ones included
  }

  // ------------------------------------------------------------------ common exit
  if (push.n_peers > 0) signal_peers_when_last(push.done_counter, push.peer_flag, push.n_peers, push.flag_value);
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) {
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) {
      }
      if (status != nullptr && atomicCAS(status, kOk, kErrBarrierTimeout) == kOk) {
        status[1] = 1000000 + blockIdx.x;
        status[2] = M;
        status[3] = N;
      }
    }
    __syncthreads();
  }
  cluster_sync_all();  // the peer may still be signalling barriers in this CTA's shared memory
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace pair

const char* make_tmap_2d(CUtensorMap* out, const void* ptr, int fmt, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                         uint32_t box_rows);
const char* make_tmap_out(CUtensorMap* out, const void* ptr, int fmt, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                          uint32_t box_rows);

template <bool A_MN, bool B_MN, bool OUT_F32, bool ACCUM, bool BIAS>
static cudaError_t launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const GemmArgs& g, int num_sms, cudaStream_t stream) {
  using namespace pair;
  auto kern = gemm_tcgen05_pair_kernel<A_MN, B_MN, OUT_F32, ACCUM, BIAS>;
  // function attributes are per device: remember which devices of this process have been set up
  static bool configured[kMaxDevices] = {};
  int dev = 0;
  if (cudaError_t e = cudaGetDevice(&dev); e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < kMaxDevices) configured[dev] = true;
  }
  const int tiles = ((g.M + 2 * BM - 1) / (2 * BM)) * ((g.N + BN - 1) / BN);
  int pairs = num_sms / 2;
  if (tiles < pairs) pairs = tiles;
  // a pushing launch stores finished sums; partial sums of a K-split tile cannot be pushed
  const int max_split = (!g.split_tail || g.push.n_peers > 0) ? 1 : 4;
  static const int group_m = [] {
    const char* e = getenv("ELF_B200_GEMM_GROUP_M");
    const int v = e ? atoi(e) : DEFAULT_GROUP_M;
    return v >= 1 && v <= 64 ? v : DEFAULT_GROUP_M;
  }();
  const Schedule sched = make_schedule(g.M, g.N, (g.K + BK - 1) / BK, pairs, max_split, group_m);
  if (sched.ksplit > 1 && !g.accumulate) {
    // K-split tiles add their partial sums to D, so D must start at zero there.  The split
    // tiles are the last ones of the tile order, all inside the row band that starts at the
    // first row of the group holding the first of them: one memset clears that band (the
    // whole tiles that share it are stored afterwards and simply overwrite the zeros).
    int m, n;
    tile_coords(sched.full_tiles, sched, &m, &n);
    const long long row_start = (long long)(m / group_m) * group_m * 2 * BM;
    const size_t esz = g.out_f32 ? 4 : 2;
    char* base = static_cast<char*>(g.d) + size_t(row_start) * size_t(g.ldd) * esz;
    const size_t rows = size_t(g.M - row_start);
    cudaError_t e = g.ldd == g.N ? cudaMemsetAsync(base, 0, rows * size_t(g.N) * esz, stream)
                                 : cudaMemset2DAsync(base, size_t(g.ldd) * esz, 0, size_t(g.N) * esz, rows, stream);
    if (e != cudaSuccess) return e;
  }
  PeerMaps peers;
  for (int p = 0; p < kMaxPeers; ++p) peers.m[p] = td;  // unused entries stay valid maps
  for (int p = 0; p < g.push.n_peers; ++p) {
    if (make_tmap_out(&peers.m[p], g.push.peer_out[p], g.out_f32 ? 2 : g.fmt, (uint64_t)g.M, (uint64_t)g.N, (uint64_t)g.ldd, g.out_f32 ? 32 : 64, BM) != nullptr)
      return cudaErrorInvalidValue;
  }
  kern<<<2 * pairs, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, td, g.d, g.bias, g.M, g.N, g.K, g.ldd, (uint32_t)g.fmt, g.alpha, max_split, group_m, g.status, g.push, peers);
  flush_bounds_record(g.status, stream);
  return cudaGetLastError();
}

template <bool A_MN, bool B_MN>
static cudaError_t dispatch_pair(const GemmArgs& g, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, int num_sms, cudaStream_t s) {
#define ELFB_LAUNCH(F32, ACC, BI) return launch_pair<A_MN, B_MN, F32, ACC, BI>(ta, tb, td, g, num_sms, s)
  if (g.out_f32) {
    if (g.accumulate) { if (g.bias) ELFB_LAUNCH(true, true, true); else ELFB_LAUNCH(true, true, false); }
    else              { if (g.bias) ELFB_LAUNCH(true, false, true); else ELFB_LAUNCH(true, false, false); }
  } else {
    if (g.accumulate) { if (g.bias) ELFB_LAUNCH(false, true, true); else ELFB_LAUNCH(false, true, false); }
    else              { if (g.bias) ELFB_LAUNCH(false, false, true); else ELFB_LAUNCH(false, false, false); }
  }
#undef ELFB_LAUNCH
}

const char* gemm_tcgen05_pair(const GemmArgs& g, int num_sms, cudaStream_t stream) {
  using namespace pair;
  if (g.M <= 0 || g.N <= 0 || g.K <= 0) return nullptr;
  CUtensorMap ta, tb;
  const char* err;
  if (g.a_mn_major) err = make_tmap_2d(&ta, g.a, g.fmt, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)g.lda, 64, BK);
  else              err = make_tmap_2d(&ta, g.a, g.fmt, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.lda, BK, BM);
  if (err) return err;
  // each CTA fetches half of the tile's B rows: one 128-row box (K-major) or two 64-wide boxes (MN-major)
  if (g.b_mn_major) err = make_tmap_2d(&tb, g.b, g.fmt, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.ldb, 64, BK);
  else              err = make_tmap_2d(&tb, g.b, g.fmt, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb, BK, BN / 2);
  if (err) return err;
  const int esz = g.out_f32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(g.d) & 15) != 0 || (g.ldd * esz) % 16 != 0) return "GEMM output must be 16-byte aligned with a 16-byte multiple row pitch";
  // output map for the TMA-store epilogue: 128-byte-wide, 128-row boxes
  CUtensorMap td;
  err = make_tmap_out(&td, g.d, g.out_f32 ? 2 : g.fmt, (uint64_t)g.M, (uint64_t)g.N, (uint64_t)g.ldd, g.out_f32 ? 32 : 64, BM);
  if (err) return err;
  cudaError_t e;
  if (g.a_mn_major && g.b_mn_major) e = dispatch_pair<true, true>(g, ta, tb, td, num_sms, stream);
  else if (!g.a_mn_major && g.b_mn_major) e = dispatch_pair<false, true>(g, ta, tb, td, num_sms, stream);
  else if (!g.a_mn_major && !g.b_mn_major) e = dispatch_pair<false, false>(g, ta, tb, td, num_sms, stream);
  else e = dispatch_pair<true, false>(g, ta, tb, td, num_sms, stream);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace elfb
