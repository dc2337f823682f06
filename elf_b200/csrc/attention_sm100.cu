// Causal GQA flash attention forward on tcgen05 / TMEM (head_dim 128, bf16).
//
// A work item is one (batch, query head, 128-row query tile).  The kernel is persistent: one
// CTA per SM walks a static list of items (heaviest first, dealt in zigzag order so that every
// CTA gets nearly the same number of key tiles).  Per 128-key tile j of an item:
//     S_j = Q K_j^T            tcgen05.mma, both operands K-major in shared memory  -> TMEM
//     P_j = exp2(S_j*c - m)    softmax warps: one thread per query row, S read with tcgen05.ld,
//                              P written to its own TMEM columns as packed bf16 with tcgen05.st
//     O  += P_j V_j            tcgen05.mma with A = P_j straight from TMEM, B = V_j (MN-major)
// Roles (384 threads): warp 0 = TMA producer for Q and K, warp 2 = TMA producer for V (two
// independent rings of 3 stages, so a late V slot never delays a K load), warp 1 = MMA issuer
// (one thread), warps 4..11 = softmax / correction / epilogue: two threads per query row, each
// owning 64 of the tile's 128 key columns (a single warp per scheduler cannot hide the
// latencies of its own dependent instructions; two can), exchanging their partial row maxima
// through shared memory.  S and P are double-buffered in
// TMEM so that Q K_{j+1}^T runs while softmax works on tile j and P_j V_j runs while softmax
// works on tile j+1; all rings and buffers keep rotating across item boundaries, so the next
// item's first loads and its first MMA overlap the current item's epilogue.  The running
// maximum is only raised (and O rescaled through TMEM) when a row's maximum grows by more
// than 2^8, which keeps exp2 in range and makes rescaling rare after the first tiles.  The
// output leaves straight from registers (each thread owns 128 bytes of a row of O).  Every
// mbarrier wait is bounded.
//
// TMEM columns: [0,128) S0, [128,256) S1, [256,384) O, [384,448) P0, [448,512) P1 (bf16 pairs).

#include <cstdint>
#include <cstdio>

#include "sm100_ptx.cuh"
#include "attention_sm100.h"

namespace elfb {

const char* make_tmap_2d(CUtensorMap* out, const void* ptr, int fmt, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                         uint32_t box_rows);

namespace attn {

constexpr int D = 128;            // head dim
constexpr int BQ = 128;           // query rows per item
constexpr int BKV = 128;          // keys per tile
constexpr int TILE_BYTES = 128 * D * 2;  // 32 KiB: two 64-column boxes of 128 rows
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int KV_STAGES = 3;
constexpr int NUM_THREADS = 384;
constexpr int XCHG_BYTES = 2 * 2 * 128 * 4;  // [parity][column half][row] partial row maxima / sums
constexpr int TMEM_COLS = 512;
__host__ __device__ constexpr int s_col(int s) { return s * 128; }
__host__ __device__ constexpr int p_col(int s) { return 384 + s * 64; }
constexpr int O_COL = 256;
constexpr size_t SMEM_BYTES = size_t(TILE_BYTES) * (1 + 2 * KV_STAGES) + XCHG_BYTES + 256;
constexpr float RESCALE_THRESHOLD = 8.0f;  // in log2 units

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct Item {
  int q_tile, head, b;
};

// Items sorted by descending key-tile count; round k of the deal runs left to right when k is
// even and right to left when odd.
struct ItemWalk {
  int n_q_tiles, n_heads, per_level, total, cta, n_ctas;
  __device__ __forceinline__ bool get(int round, Item* it) const {
    const int idx = round * n_ctas + ((round & 1) ? (n_ctas - 1 - cta) : cta);
    if (idx >= total) return false;
    const int level = idx / per_level;
    const int rem = idx - level * per_level;
    it->q_tile = n_q_tiles - 1 - level;
    it->head = rem % n_heads;
    it->b = rem / n_heads;
    return true;
  }
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tmap_qkv, __nv_bfloat16* __restrict__ out, float* __restrict__ lse, int batch, int seq, int n_heads,
                     int n_kv_heads, float scale_log2, int* __restrict__ status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = smem_u32(smem_raw);
  if ((smem_base & 1023u) != 0) {  // the 128-byte swizzle needs 1024-byte aligned tiles
    if (threadIdx.x == 0 && status != nullptr && atomicCAS(status, kOk, kErrBadShape) == kOk) status[1] = 2900000;
    return;
  }
  uint8_t* smem_aligned = smem_raw;
  const uint32_t q_smem = smem_base;
  auto k_smem = [&](int s) { return smem_base + TILE_BYTES * (1 + s); };
  auto v_smem = [&](int s) { return smem_base + TILE_BYTES * (1 + KV_STAGES + s); };
  float* xchg = reinterpret_cast<float*>(smem_aligned + size_t(TILE_BYTES) * (1 + 2 * KV_STAGES));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_aligned + size_t(TILE_BYTES) * (1 + 2 * KV_STAGES) + XCHG_BYTES);
  const uint32_t bar0 = smem_u32(bars);
  enum {
    Q_FULL = 0, Q_EMPTY = 1, K_FULL = 2, K_EMPTY = K_FULL + KV_STAGES, V_FULL = K_EMPTY + KV_STAGES, V_EMPTY = V_FULL + KV_STAGES,
    S_FULL = V_EMPTY + KV_STAGES, P_FULL = S_FULL + 2, PV_DONE = P_FULL + 2, O_FINAL = PV_DONE + 2, N_BARS = O_FINAL + 1
  };
  auto bar = [&](int slot) { return bar0 + 8u * slot; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + N_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* pair_seq = reinterpret_cast<volatile int*>(tmem_slot + 2);  // [8]: exchanges published by each softmax warp

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  ItemWalk walk;
  walk.n_q_tiles = seq / BQ;
  walk.n_heads = n_heads;
  walk.per_level = n_heads * batch;
  walk.total = walk.per_level * walk.n_q_tiles;
  walk.cta = blockIdx.x;
  walk.n_ctas = gridDim.x;
  const int group = n_heads / n_kv_heads;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int w = 0; w < 8; ++w) pair_seq[w] = 0;
    mbar_init(bar(Q_FULL), 1);
    mbar_init(bar(Q_EMPTY), 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(bar(K_FULL + s), 1);
      mbar_init(bar(K_EMPTY + s), 1);
      mbar_init(bar(V_FULL + s), 1);
      mbar_init(bar(V_EMPTY + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(S_FULL + s), 1);
      mbar_init(bar(P_FULL + s), 8);  // one arrival per softmax warp
      mbar_init(bar(PV_DONE + s), 1);
    }
    mbar_init(bar(O_FINAL), 1);
    fence_barrier_init();
    prefetch_tensormap(&tmap_qkv);
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
    // ------------------------------------------------------------------ TMA producer: Q and K
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Item it;
      for (int round = 0; ok && walk.get(round, &it); ++round) {
        const int q_row0 = it.b * seq + it.q_tile * BQ;
        const int q_col = it.head * D;
        const int k_col = (n_heads + it.head / group) * D;
        // the previous item's last Q K^T has read the Q tile
        if (round > 0 && !mbar_wait(bar(Q_EMPTY), uint32_t(round - 1) & 1u, abort_flag)) break;
        mbar_arrive_expect_tx(bar(Q_FULL), TILE_BYTES);
        tma_load_2d(q_smem, &tmap_qkv, bar(Q_FULL), q_col, q_row0);
        tma_load_2d(q_smem + HALF_BYTES, &tmap_qkv, bar(Q_FULL), q_col + 64, q_row0);
        for (int j = 0; j <= it.q_tile; ++j) {
          if (!mbar_wait(bar(K_EMPTY + stage), phase ^ 1u, abort_flag)) { ok = false; break; }
          const int row0 = it.b * seq + j * BKV;
          mbar_arrive_expect_tx(bar(K_FULL + stage), TILE_BYTES);
          tma_load_2d(k_smem(stage), &tmap_qkv, bar(K_FULL + stage), k_col, row0);
          tma_load_2d(k_smem(stage) + HALF_BYTES, &tmap_qkv, bar(K_FULL + stage), k_col + 64, row0);
          if (++stage == KV_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    // ------------------------------------------------------------------ TMA producer: V
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Item it;
      for (int round = 0; ok && walk.get(round, &it); ++round) {
        const int v_col = (n_heads + n_kv_heads + it.head / group) * D;
        for (int j = 0; j <= it.q_tile; ++j) {
          if (!mbar_wait(bar(V_EMPTY + stage), phase ^ 1u, abort_flag)) { ok = false; break; }
          const int row0 = it.b * seq + j * BKV;
          mbar_arrive_expect_tx(bar(V_FULL + stage), TILE_BYTES);
          tma_load_2d(v_smem(stage), &tmap_qkv, bar(V_FULL + stage), v_col, row0);
          tma_load_2d(v_smem(stage) + HALF_BYTES, &tmap_qkv, bar(V_FULL + stage), v_col + 64, row0);
          if (++stage == KV_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc_f16(1u, BQ, BKV, 0u, 0u);  // S[128 q,128 k] = Q (K-major) x K (K-major)
      const uint32_t idesc_pv = make_idesc_f16(1u, BQ, D, 0u, 1u);    // O[128 q,128 d] = P (TMEM) x V (MN-major)
      int k_stage = 0, v_stage = 0;
      uint32_t k_phase = 0, v_phase = 0;
      int g = 0;  // tiles issued so far over all items: S / P buffer = g & 1
      bool ok = true;
      // P_t V_t for the tile with running index t (t_local = its index inside the item)
      auto issue_pv = [&](int t, int t_local) -> bool {
        const int s = t & 1;
        if (!mbar_wait(bar(P_FULL + s), uint32_t(t >> 1) & 1u, abort_flag)) return false;
        if (!mbar_wait(bar(V_FULL + v_stage), v_phase, abort_flag)) return false;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          // A: P, bf16 pairs in 64 TMEM columns: 16 keys = 8 columns
          // B: V, two 64-wide (d) boxes of 128 key rows; 16 keys = 16 rows = 2048 bytes
          const uint64_t db = make_smem_desc_sw128(v_smem(v_stage) + kk * 2048, HALF_BYTES, 1024);
          umma_ts(tmem_base + O_COL, tmem_base + p_col(s) + kk * 8, db, idesc_pv, (t_local | kk) ? 1u : 0u);
        }
        umma_commit(bar(V_EMPTY + v_stage));
        umma_commit(bar(PV_DONE + s));
        if (++v_stage == KV_STAGES) { v_stage = 0; v_phase ^= 1u; }
        return true;
      };
      Item it;
      for (int round = 0; ok && walk.get(round, &it); ++round) {
        const int n_kv = it.q_tile + 1;
        if (!mbar_wait(bar(Q_FULL), uint32_t(round) & 1u, abort_flag)) break;
        for (int j = 0; j < n_kv; ++j) {
          const int s = (g + j) & 1;
          if (!mbar_wait(bar(K_FULL + k_stage), k_phase, abort_flag)) { ok = false; break; }
          // S buffer s was last read by the softmax of the tile two back, which the P V issue of that tile waited for
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            // K-major tiles: two 64-element (128 B) column halves, 16 KiB apart; 16 elements = 32 B
            const uint32_t off = uint32_t(kk >> 2) * HALF_BYTES + uint32_t(kk & 3) * 32u;
            const uint64_t da = make_smem_desc_sw128(q_smem + off, 0, 1024);
            const uint64_t db = make_smem_desc_sw128(k_smem(k_stage) + off, 0, 1024);
            umma_ss(tmem_base + s_col(s), da, db, idesc_qk, kk ? 1u : 0u);
          }
          umma_commit(bar(K_EMPTY + k_stage));
          umma_commit(bar(S_FULL + s));
          if (j == n_kv - 1) umma_commit(bar(Q_EMPTY));
          if (++k_stage == KV_STAGES) { k_stage = 0; k_phase ^= 1u; }
          if (j >= 1 && !issue_pv(g + j - 1, j - 1)) { ok = false; break; }
        }
        if (!ok || !issue_pv(g + n_kv - 1, n_kv - 1)) { ok = false; break; }
        umma_commit(bar(O_FINAL));
        g += n_kv;
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    const int quarter = warp & 3;                 // TMEM lanes [32*quarter, +32)
    const int half = (warp - 4) >> 2;             // key columns [64*half, +64) of every tile
    const int r = quarter * 32 + lane;            // query row inside the tile
    const uint32_t lane_off = uint32_t(quarter * 32) << 16;
    const int my_slot = warp - 4, partner_slot = (warp - 4) ^ 4;  // the two warps that share these rows
    int g = 0;
    int xc = 0;  // exchanges so far
    bool ok = true;
    // Both threads of a row publish a value and read the partner's.  Values are double-buffered by
    // the parity of the exchange count; a warp announces its n-th values by writing n to its
    // sequence word and waits (bounded) for the partner warp's.  A warp can only overwrite a buffer
    // two exchanges later, which it reaches after the partner has announced the exchange in
    // between, that is after the partner has finished reading this one.
    auto exchange = [&](float mine, float* theirs) -> bool {
      float* buf = xchg + (xc & 1) * 256;
      buf[half * 128 + r] = mine;
      ++xc;
      __threadfence_block();
      __syncwarp();
      if (lane == 0) pair_seq[my_slot] = xc;
      if (pair_seq[partner_slot] < xc) {
        const unsigned long long t0 = globaltimer_ns();
        for (uint32_t spin = 1; pair_seq[partner_slot] < xc; ++spin) {
          if ((spin & 0xffu) == 0) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > kWaitLimitNs) {
              *abort_flag = 1;
              return false;
            }
          }
        }
      }
      __threadfence_block();
      *theirs = buf[(half ^ 1) * 128 + r];
      return true;
    };
    Item it;
    for (int round = 0; ok && walk.get(round, &it); ++round) {
      const int n_kv = it.q_tile + 1;
      float m_ref = -INFINITY;  // reference maximum (scaled, log2 domain) the stored exponentials refer to
      float l = 0.f;            // this thread's share of the running sum of exp2(x * c - m_ref)
      for (int j = 0; j < n_kv; ++j) {
        const int t = g + j;
        const int s = t & 1;
        if (!mbar_wait(bar(S_FULL + s), uint32_t(t >> 1) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        // this thread's 64 raw scores: two loads in flight, one wait
        uint32_t v[2][32];
#pragma unroll
        for (int c = 0; c < 2; ++c) tmem_ld_32x32b_x32(tmem_base + lane_off + s_col(s) + half * 64 + c * 32, v[c]);
        tmem_ld_wait();
        if (j == it.q_tile) {  // diagonal tile: keys after the query are masked
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (half * 64 + c * 32 + i > r) v[c][i] = 0xff800000u;  // -inf
        }
        float mx4[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) mx4[q] = __uint_as_float(v[q >> 1][(q & 1) * 16]);
#pragma unroll
        for (int i = 1; i < 16; ++i)
#pragma unroll
          for (int q = 0; q < 4; ++q) mx4[q] = fmaxf(mx4[q], __uint_as_float(v[q >> 1][(q & 1) * 16 + i]));
        const float mine = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        float theirs;
        if (!exchange(mine, &theirs)) { ok = false; break; }
        const float mx = fmaxf(mine, theirs) * scale_log2;
        // raise the reference maximum only when it pays (always on the first tile); both
        // threads of a row see the same numbers and take the same decision
        const bool raise = mx > m_ref + RESCALE_THRESHOLD;
        if (__any_sync(0xffffffffu, raise)) {
          const float m_new = raise ? mx : m_ref;
          const float factor = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m_new);
          l *= factor;
          m_ref = m_new;
          if (j > 0) {
            // O holds the sum up to tile j-1 once P_{j-1} V_{j-1} has completed
            if (!mbar_wait(bar(PV_DONE + ((t - 1) & 1)), uint32_t((t - 1) >> 1) & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t o_addr = tmem_base + lane_off + O_COL + half * 64;
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {  // rare after the first tiles: kept rolled to save registers
              uint32_t o[32];
              tmem_ld_32x32b_x32(o_addr + c * 32, o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
              tmem_st_32x32b_x32(o_addr + c * 32, o);
            }
            tmem_st_wait();
          }
        }
        // P buffer s was last read by the P V product of the tile two back
        if (t >= 2 && !mbar_wait(bar(PV_DONE + s), uint32_t((t - 2) >> 1) & 1u, abort_flag)) { ok = false; break; }
        const float neg_m = -m_ref;
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(v[i >> 4][(2 * i) & 31]), scale_log2, neg_m));
          const float p1 = fast_exp2(fmaf(__uint_as_float(v[i >> 4][(2 * i + 1) & 31]), scale_log2, neg_m));
          sum4[i & 3] += p0 + p1;
          pk[i] = pack_bf16x2(p0, p1);
        }
        tmem_st_32x32b_x32(tmem_base + lane_off + p_col(s) + half * 32, pk);
        l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(P_FULL + s));
      }
      if (!ok) break;
      g += n_kv;
      // ---- epilogue: O / l -> bf16, straight from registers (each thread owns 128 bytes of a row)
      float l_other;
      if (!exchange(l, &l_other)) break;
      const float l_row = l + l_other;
      if (!mbar_wait(bar(O_FINAL), uint32_t(round) & 1u, abort_flag)) break;
      tc_fence_after_sync();
      const float inv_l = 1.f / l_row;
      const size_t token = size_t(it.b) * seq + size_t(it.q_tile) * BQ + r;
      uint4* dst = reinterpret_cast<uint4*>(out + (token * n_heads + it.head) * D + half * 64);
      const uint32_t o_addr = tmem_base + lane_off + O_COL + half * 64;
      uint32_t o[2][32];
#pragma unroll
      for (int c = 0; c < 2; ++c) tmem_ld_32x32b_x32(o_addr + c * 32, o[c]);
      tmem_ld_wait();
      // O may be overwritten by the next item's first P V from here on: that product waits for this
      // warp's next arrival on P_FULL, which program order puts after these loads
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(o[c][8 * q]) * inv_l, __uint_as_float(o[c][8 * q + 1]) * inv_l);
          w.y = pack_bf16x2(__uint_as_float(o[c][8 * q + 2]) * inv_l, __uint_as_float(o[c][8 * q + 3]) * inv_l);
          w.z = pack_bf16x2(__uint_as_float(o[c][8 * q + 4]) * inv_l, __uint_as_float(o[c][8 * q + 5]) * inv_l);
          w.w = pack_bf16x2(__uint_as_float(o[c][8 * q + 6]) * inv_l, __uint_as_float(o[c][8 * q + 7]) * inv_l);
          dst[c * 4 + q] = w;
        }
      if (half == 0) lse[(size_t(it.b) * n_heads + it.head) * seq + it.q_tile * BQ + r] = (m_ref + log2f(l_row)) * 0.6931471805599453f;
    }
  }

  // ------------------------------------------------------------------ common exit
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) {
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) {
      }
      if (status != nullptr && atomicCAS(status, kOk, kErrBarrierTimeout) == kOk) {
        status[1] = 2000000 + blockIdx.x;
        status[2] = seq;
        status[3] = n_heads;
      }
    }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace attn

const char* attention_forward(const AttnArgs& a, cudaStream_t stream) {
  using namespace attn;
  if (a.batch <= 0 || a.seq <= 0) return nullptr;
  if (a.seq % BQ != 0) return "attention: sequence length must be a multiple of 128";
  if (a.n_kv_heads <= 0 || a.n_heads % a.n_kv_heads != 0) return "attention: query heads must be a multiple of key/value heads";
  if ((reinterpret_cast<uintptr_t>(a.out) & 15) != 0) return "attention: output must be 16-byte aligned";
  const uint64_t rows = uint64_t(a.batch) * a.seq;
  const uint64_t pitch = uint64_t(a.n_heads + 2 * a.n_kv_heads) * D;
  CUtensorMap tq;
  const char* err = make_tmap_2d(&tq, a.qkv, 1, rows, pitch, pitch, 64, 128);
  if (err) return err;
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return "attention: cannot query the device";
    if (cudaFuncSetAttribute(attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES) != cudaSuccess) {
      num_sms = 0;
      return "attention: cannot raise the shared memory limit";
    }
  }
  const float scale = a.scale > 0.f ? a.scale : 0.08838834764831845f;
  const long long items = (long long)(a.seq / BQ) * a.n_heads * a.batch;
  const int grid = int(items < num_sms ? items : num_sms);
  attention_fwd_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tq, static_cast<__nv_bfloat16*>(a.out), a.lse, a.batch, a.seq, a.n_heads, a.n_kv_heads,
                                                                  scale * 1.4426950408889634f, a.status);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace elfb
