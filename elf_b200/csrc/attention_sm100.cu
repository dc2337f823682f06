// Causal GQA flash attention forward on tcgen05 / TMEM (head_dim 128, bf16).
//
// A work item is a PAIR of 128-row query tiles that share their key/value head, so that every
// K and V tile fetched from L2 feeds two score and two output products (with one query tile per
// CTA the kernel is bound by L2 -> shared-memory bandwidth, not by the tensor pipe):
//   * grouped-query models with an even group size pair two query heads of one KV group at the
//     same query tile (identical masks and key ranges);
//   * otherwise (multi-head attention) two consecutive query tiles of one head are paired; the
//     upper one sees one key tile more than the lower one.
// The kernel is persistent: one CTA per SM walks a static list of items (heaviest first, dealt
// in zigzag order so that every CTA gets nearly the same number of key tiles).  Per sub-item
// X in {A, B} and 128-key tile j:
//     S_X = Q_X K_j^T          tcgen05.mma, both operands K-major in shared memory  -> TMEM
//     P_X = exp2(S_X*c - m)    softmax warps of X: one thread per query row, S read with
//                              tcgen05.ld, P written over S as packed bf16 with tcgen05.st
//     O_X += P_X V_j           tcgen05.mma with A = P_X straight from TMEM, B = V_j (MN-major)
// Roles (384 threads): warp 0 = TMA producer for Q and K (3-stage K ring), warp 2 = TMA
// producer for V (2-stage ring), warp 1 = MMA issuer (one thread), warps 4..7 = softmax /
// correction / epilogue of A, warps 8..11 = the same for B.  The issuer alternates between the
// sub-items (P_A V, Q_A K_next, P_B V, Q_B K_next), so the tensor pipe works for one sub-item while
// the other one's softmax runs, and each scheduler has two independent softmax warps whose
// latencies hide each other.  The running maximum is only raised (and O rescaled through
// TMEM) when a row's maximum grows by more than 2^8, which keeps exp2 in range and makes
// rescaling rare after the first tiles.  The output leaves straight from registers (each
// thread owns a 256-byte row of O).  Every mbarrier wait is bounded.
//
// TMEM columns: [0,128) S_A (P_A in its first 64), [128,256) S_B / P_B, [256,384) O_A, [384,512) O_B.

#include <cstdint>
#include <cstdio>

#include "sm100_ptx.cuh"
#include "attention_sm100.h"

namespace elfb {

const char* make_tmap_2d(CUtensorMap* out, const void* ptr, int fmt, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                         uint32_t box_rows);

namespace attn {

constexpr int D = 128;            // head dim
constexpr int BQ = 128;           // query rows per sub-item
constexpr int BKV = 128;          // keys per tile
constexpr int TILE_BYTES = 128 * D * 2;  // 32 KiB: two 64-column boxes of 128 rows
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int K_STAGES = 3;
constexpr int V_STAGES = 2;
constexpr int NUM_THREADS = 384;
constexpr int TMEM_COLS = 512;
__host__ __device__ constexpr int s_col(int x) { return x * 128; }
__host__ __device__ constexpr int o_col(int x) { return 256 + x * 128; }
constexpr size_t SMEM_BYTES = size_t(TILE_BYTES) * (2 + K_STAGES + V_STAGES) + 256;
constexpr float RESCALE_THRESHOLD = 8.0f;  // in log2 units

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct Item {
  int b, kv_head;
  int q_tile[2], head[2], n_kv[2];  // n_kv[0] <= n_kv[1]; n_kv[0] == 0: sub-item A is absent
};

// Items sorted by descending key-tile count; round k of the deal runs left to right when k is
// even and right to left when odd.
struct ItemWalk {
  int n_q_tiles, n_heads, group, per_level, total, cta, n_ctas;
  bool pair_heads;
  __device__ __forceinline__ void init(int seq, int heads, int kv_heads, int batch) {
    n_q_tiles = seq / BQ;
    n_heads = heads;
    group = heads / kv_heads;
    pair_heads = (group % 2) == 0;
    per_level = pair_heads ? batch * (heads / 2) : batch * heads;
    total = per_level * (pair_heads ? n_q_tiles : (n_q_tiles + 1) / 2);
    cta = blockIdx.x;
    n_ctas = gridDim.x;
  }
  __device__ __forceinline__ bool get(int round, Item* it) const {
    const int idx = round * n_ctas + ((round & 1) ? (n_ctas - 1 - cta) : cta);
    if (idx >= total) return false;
    const int level = idx / per_level;
    const int rem = idx - level * per_level;
    if (pair_heads) {
      const int hp = rem % (n_heads / 2);
      it->b = rem / (n_heads / 2);
      it->head[0] = 2 * hp;
      it->head[1] = 2 * hp + 1;
      it->q_tile[0] = it->q_tile[1] = n_q_tiles - 1 - level;
      it->n_kv[0] = it->n_kv[1] = it->q_tile[0] + 1;
    } else {
      it->b = rem / n_heads;
      it->head[0] = it->head[1] = rem % n_heads;
      it->q_tile[1] = n_q_tiles - 1 - 2 * level;
      it->q_tile[0] = it->q_tile[1] - 1;
      it->n_kv[1] = it->q_tile[1] + 1;
      it->n_kv[0] = it->q_tile[1];  // 0 when the upper tile is the first one: no lower tile
    }
    it->kv_head = it->head[0] / group;
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
  auto q_smem = [&](int x) { return smem_base + TILE_BYTES * x; };
  auto k_smem = [&](int s) { return smem_base + TILE_BYTES * (2 + s); };
  auto v_smem = [&](int s) { return smem_base + TILE_BYTES * (2 + K_STAGES + s); };
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + size_t(TILE_BYTES) * (2 + K_STAGES + V_STAGES));
  const uint32_t bar0 = smem_u32(bars);
  enum {
    Q_FULL = 0, Q_EMPTY = 2, K_FULL = 4, K_EMPTY = K_FULL + K_STAGES, V_FULL = K_EMPTY + K_STAGES, V_EMPTY = V_FULL + V_STAGES,
    S_FULL = V_EMPTY + V_STAGES, P_FULL = S_FULL + 2, PV_DONE = P_FULL + 2, O_FINAL = PV_DONE + 2, N_BARS = O_FINAL + 2
  };
  auto bar = [&](int slot) { return bar0 + 8u * slot; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + N_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  ItemWalk walk;
  walk.init(seq, n_heads, n_kv_heads, batch);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int x = 0; x < 2; ++x) {
      mbar_init(bar(Q_FULL + x), 1);
      mbar_init(bar(Q_EMPTY + x), 1);
      mbar_init(bar(S_FULL + x), 1);
      mbar_init(bar(P_FULL + x), 4);  // one arrival per softmax warp of the sub-item
      mbar_init(bar(PV_DONE + x), 1);
      mbar_init(bar(O_FINAL + x), 1);
    }
    for (int s = 0; s < K_STAGES; ++s) {
      mbar_init(bar(K_FULL + s), 1);
      mbar_init(bar(K_EMPTY + s), 1);
    }
    for (int s = 0; s < V_STAGES; ++s) {
      mbar_init(bar(V_FULL + s), 1);
      mbar_init(bar(V_EMPTY + s), 1);
    }
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
      int kc = 0;               // K tiles requested so far: stage kc % K_STAGES
      int q_uses[2] = {0, 0};   // items in which each Q buffer has been used
      bool ok = true;
      Item it;
      for (int round = 0; ok && walk.get(round, &it); ++round) {
        for (int x = 0; x < 2 && ok; ++x) {
          if (it.n_kv[x] == 0) continue;
          // the previous user's last Q K^T has read this Q buffer
          if (q_uses[x] > 0 && !mbar_wait(bar(Q_EMPTY + x), uint32_t(q_uses[x] - 1) & 1u, abort_flag)) { ok = false; break; }
          ++q_uses[x];
          const int row0 = it.b * seq + it.q_tile[x] * BQ;
          mbar_arrive_expect_tx(bar(Q_FULL + x), TILE_BYTES);
          tma_load_2d(q_smem(x), &tmap_qkv, bar(Q_FULL + x), it.head[x] * D, row0);
          tma_load_2d(q_smem(x) + HALF_BYTES, &tmap_qkv, bar(Q_FULL + x), it.head[x] * D + 64, row0);
        }
        const int k_col = (n_heads + it.kv_head) * D;
        for (int j = 0; j < it.n_kv[1] && ok; ++j, ++kc) {
          const int stage = kc % K_STAGES;
          if (!mbar_wait(bar(K_EMPTY + stage), (uint32_t(kc / K_STAGES) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
          const int row0 = it.b * seq + j * BKV;
          mbar_arrive_expect_tx(bar(K_FULL + stage), TILE_BYTES);
          tma_load_2d(k_smem(stage), &tmap_qkv, bar(K_FULL + stage), k_col, row0);
          tma_load_2d(k_smem(stage) + HALF_BYTES, &tmap_qkv, bar(K_FULL + stage), k_col + 64, row0);
        }
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    // ------------------------------------------------------------------ TMA producer: V
    if (lane == 0) {
      int vc = 0;
      bool ok = true;
      Item it;
      for (int round = 0; ok && walk.get(round, &it); ++round) {
        const int v_col = (n_heads + n_kv_heads + it.kv_head) * D;
        for (int j = 0; j < it.n_kv[1]; ++j, ++vc) {
          const int stage = vc % V_STAGES;
          if (!mbar_wait(bar(V_EMPTY + stage), (uint32_t(vc / V_STAGES) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
          const int row0 = it.b * seq + j * BKV;
          mbar_arrive_expect_tx(bar(V_FULL + stage), TILE_BYTES);
          tma_load_2d(v_smem(stage), &tmap_qkv, bar(V_FULL + stage), v_col, row0);
          tma_load_2d(v_smem(stage) + HALF_BYTES, &tmap_qkv, bar(V_FULL + stage), v_col + 64, row0);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc_f16(1u, BQ, BKV, 0u, 0u);  // S[128 q,128 k] = Q (K-major) x K (K-major)
      const uint32_t idesc_pv = make_idesc_f16(1u, BQ, D, 0u, 1u);    // O[128 q,128 d] = P (TMEM) x V (MN-major)
      int kc = 0, vc = 0;        // K / V tiles consumed before this item
      int tiles[2] = {0, 0};     // tiles of each sub-item issued before this item: parity of S_FULL / P_FULL / PV_DONE
      int q_uses[2] = {0, 0};
      bool ok = true;
      // S_x = Q_x K^T for K tile number k_idx (running index)
      auto issue_qk = [&](int x, int k_idx) -> bool {
        const int stage = k_idx % K_STAGES;
        if (!mbar_wait(bar(K_FULL + stage), uint32_t(k_idx / K_STAGES) & 1u, abort_flag)) return false;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          // K-major tiles: two 64-element (128 B) column halves, 16 KiB apart; 16 elements = 32 B
          const uint32_t off = uint32_t(kk >> 2) * HALF_BYTES + uint32_t(kk & 3) * 32u;
          const uint64_t da = make_smem_desc_sw128(q_smem(x) + off, 0, 1024);
          const uint64_t db = make_smem_desc_sw128(k_smem(stage) + off, 0, 1024);
          umma_ss(tmem_base + s_col(x), da, db, idesc_qk, kk ? 1u : 0u);
        }
        umma_commit(bar(S_FULL + x));
        return true;
      };
      // O_x (+)= P_x V for V tile number v_idx; t = running tile index of the sub-item
      auto issue_pv = [&](int x, int v_idx, int t, bool first) -> bool {
        if (!mbar_wait(bar(P_FULL + x), uint32_t(t) & 1u, abort_flag)) return false;
        const int stage = v_idx % V_STAGES;
        if (!mbar_wait(bar(V_FULL + stage), uint32_t(v_idx / V_STAGES) & 1u, abort_flag)) return false;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          // A: P, bf16 pairs in 64 TMEM columns: 16 keys = 8 columns
          // B: V, two 64-wide (d) boxes of 128 key rows; 16 keys = 16 rows = 2048 bytes
          const uint64_t db = make_smem_desc_sw128(v_smem(stage) + kk * 2048, HALF_BYTES, 1024);
          umma_ts(tmem_base + o_col(x), tmem_base + s_col(x) + kk * 8, db, idesc_pv, (!first || kk) ? 1u : 0u);
        }
        umma_commit(bar(PV_DONE + x));
        return true;
      };
      Item it;
      for (int round = 0; ok && walk.get(round, &it); ++round) {
        const int n_a = it.n_kv[0], n_b = it.n_kv[1];
        for (int x = 0; x < 2 && ok; ++x) {
          if (it.n_kv[x] == 0) continue;
          if (!mbar_wait(bar(Q_FULL + x), uint32_t(q_uses[x]) & 1u, abort_flag)) ok = false;
          ++q_uses[x];
        }
        if (!ok) break;
        // first key tile of both sub-items
        if (n_a > 0) {
          if (!issue_qk(0, kc)) break;
          if (n_a == 1) umma_commit(bar(Q_EMPTY + 0));
        }
        if (!issue_qk(1, kc)) break;
        umma_commit(bar(K_EMPTY + kc % K_STAGES));
        if (n_b == 1) umma_commit(bar(Q_EMPTY + 1));
        for (int j = 0; j < n_b; ++j) {
          if (j < n_a) {
            if (!issue_pv(0, vc + j, tiles[0] + j, j == 0)) { ok = false; break; }
            if (j == n_a - 1) umma_commit(bar(O_FINAL + 0));
            if (j + 1 < n_a) {
              // S_A / P_A are free again once the product just issued has run: same thread, in order
              if (!issue_qk(0, kc + j + 1)) { ok = false; break; }
              if (j + 2 == n_a) umma_commit(bar(Q_EMPTY + 0));
            }
          }
          if (!issue_pv(1, vc + j, tiles[1] + j, j == 0)) { ok = false; break; }
          umma_commit(bar(V_EMPTY + (vc + j) % V_STAGES));
          if (j == n_b - 1) umma_commit(bar(O_FINAL + 1));
          if (j + 1 < n_b) {
            if (!issue_qk(1, kc + j + 1)) { ok = false; break; }
            umma_commit(bar(K_EMPTY + (kc + j + 1) % K_STAGES));
            if (j + 2 == n_b) umma_commit(bar(Q_EMPTY + 1));
          }
        }
        kc += n_b;
        vc += n_b;
        tiles[0] += n_a;
        tiles[1] += n_b;
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax / correction / epilogue of sub-item x
    const int x = (warp - 4) >> 2;
    const int quarter = warp & 3;                 // TMEM lanes [32*quarter, +32)
    const int r = quarter * 32 + lane;            // query row inside the tile
    const uint32_t lane_off = uint32_t(quarter * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_off + s_col(x);
    const uint32_t o_addr = tmem_base + lane_off + o_col(x);
    int tiles = 0;   // tiles of this sub-item handled in earlier items
    int uses = 0;    // earlier items in which this sub-item was present
    bool ok = true;
    Item it;
    for (int round = 0; ok && walk.get(round, &it); ++round) {
      const int n_kv = it.n_kv[x];
      if (n_kv == 0) continue;
      const int diag = it.q_tile[x];
      float m_ref = -INFINITY;  // reference maximum (scaled, log2 domain) the stored exponentials refer to
      float l = 0.f;            // running sum of exp2(s * c - m_ref)
      for (int j = 0; j < n_kv; ++j) {
        const int t = tiles + j;
        if (!mbar_wait(bar(S_FULL + x), uint32_t(t) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        // pass 1: row maximum.  Columns 64..127 are read again in pass 2; columns 0..63 stay in registers.
        uint32_t lo[2][32], hi[2][32];
        tmem_ld_32x32b_x32(s_addr + 64, hi[0]);
        tmem_ld_32x32b_x32(s_addr + 96, hi[1]);
        tmem_ld_32x32b_x32(s_addr, lo[0]);
        tmem_ld_32x32b_x32(s_addr + 32, lo[1]);
        tmem_ld_wait();
        if (j == diag) {  // diagonal tile: keys after the query are masked
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (c * 32 + i > r) lo[c][i] = 0xff800000u;  // -inf
              if (64 + c * 32 + i > r) hi[c][i] = 0xff800000u;
            }
        }
        float mx8[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          mx8[q] = __uint_as_float(lo[q >> 1][(q & 1) * 16]);
          mx8[4 + q] = __uint_as_float(hi[q >> 1][(q & 1) * 16]);
        }
#pragma unroll
        for (int i = 1; i < 16; ++i)
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            mx8[q] = fmaxf(mx8[q], __uint_as_float(lo[q >> 1][(q & 1) * 16 + i]));
            mx8[4 + q] = fmaxf(mx8[4 + q], __uint_as_float(hi[q >> 1][(q & 1) * 16 + i]));
          }
        const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])), fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7]))) * scale_log2;
        // raise the reference maximum only when it pays (always on the first tile)
        const bool raise = mx > m_ref + RESCALE_THRESHOLD;
        if (__any_sync(0xffffffffu, raise)) {
          const float m_new = raise ? mx : m_ref;
          const float factor = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m_new);
          l *= factor;
          m_ref = m_new;
          if (j > 0) {
            // O holds the sum up to tile j-1 once P_{j-1} V_{j-1} has completed
            if (!mbar_wait(bar(PV_DONE + x), uint32_t(t - 1) & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {  // rare after the first tiles: kept rolled to save registers
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
        // pass 2: exponentials, written over the scores as packed bf16 (keys 2i, 2i+1 -> column i)
        const float neg_m = -m_ref;
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        {
          uint32_t pk[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(lo[i >> 4][(2 * i) & 31]), scale_log2, neg_m));
            const float p1 = fast_exp2(fmaf(__uint_as_float(lo[i >> 4][(2 * i + 1) & 31]), scale_log2, neg_m));
            sum4[i & 3] += p0 + p1;
            pk[i] = pack_bf16x2(p0, p1);
          }
          tmem_st_32x32b_x32(s_addr, pk);  // covers score columns 0..31, already in registers
        }
        {
          uint32_t pk[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(hi[i >> 4][(2 * i) & 31]), scale_log2, neg_m));
            const float p1 = fast_exp2(fmaf(__uint_as_float(hi[i >> 4][(2 * i + 1) & 31]), scale_log2, neg_m));
            sum4[i & 3] += p0 + p1;
            pk[i] = pack_bf16x2(p0, p1);
          }
          tmem_st_32x32b_x32(s_addr + 32, pk);  // covers score columns 32..63, already in registers
        }
        l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(P_FULL + x));
      }
      if (!ok) break;
      tiles += n_kv;
      // ---- epilogue: O / l -> bf16, straight from registers (each thread owns one 256-byte row)
      if (!mbar_wait(bar(O_FINAL + x), uint32_t(uses) & 1u, abort_flag)) break;
      ++uses;
      tc_fence_after_sync();
      const float inv_l = 1.f / l;
      const size_t token = size_t(it.b) * seq + size_t(it.q_tile[x]) * BQ + r;
      uint4* dst = reinterpret_cast<uint4*>(out + (token * n_heads + it.head[x]) * D);
      // O may be overwritten by the next item's first P V once these loads are done: that product
      // waits for this warp's next arrival on P_FULL, which program order puts after them
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(o_addr + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(o[8 * q]) * inv_l, __uint_as_float(o[8 * q + 1]) * inv_l);
          w.y = pack_bf16x2(__uint_as_float(o[8 * q + 2]) * inv_l, __uint_as_float(o[8 * q + 3]) * inv_l);
          w.z = pack_bf16x2(__uint_as_float(o[8 * q + 4]) * inv_l, __uint_as_float(o[8 * q + 5]) * inv_l);
          w.w = pack_bf16x2(__uint_as_float(o[8 * q + 6]) * inv_l, __uint_as_float(o[8 * q + 7]) * inv_l);
          dst[c * 4 + q] = w;
        }
      }
      lse[(size_t(it.b) * n_heads + it.head[x]) * seq + it.q_tile[x] * BQ + r] = (m_ref + log2f(l)) * 0.6931471805599453f;
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
  // SM count and function attributes are per device
  static int sms_of[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return "attention: cannot query the device";
  if (sms_of[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return "attention: cannot query the device";
    if (cudaFuncSetAttribute(attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES) != cudaSuccess)
      return "attention: cannot raise the shared memory limit";
    sms_of[dev] = n;
  }
  const int num_sms = sms_of[dev];
  const float scale = a.scale > 0.f ? a.scale : 0.08838834764831845f;
  const int group = a.n_heads / a.n_kv_heads, n_q = a.seq / BQ;
  const long long items = group % 2 == 0 ? (long long)n_q * (a.n_heads / 2) * a.batch : (long long)((n_q + 1) / 2) * a.n_heads * a.batch;
  const int grid = int(items < num_sms ? items : num_sms);
  attention_fwd_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tq, static_cast<__nv_bfloat16*>(a.out), a.lse, a.batch, a.seq, a.n_heads, a.n_kv_heads,
                                                                  scale * 1.4426950408889634f, a.status);
  flush_bounds_record(a.status, stream);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace elfb
