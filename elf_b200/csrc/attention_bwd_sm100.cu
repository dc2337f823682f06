// Causal GQA flash attention backward on tcgen05 / TMEM (head_dim 128, bf16).
//
// Three launches:
//   attn_bwd_prepare   delta[b,h,s] = sum_d O*dO and lse2 = lse*log2(e)      (one warp per row)
//   attn_bwd_kernel    dK, dV (written as bf16) and dQ (added into an fp32 accumulator)
//   attn_bwd_finish    dQ accumulator -> bf16 into the packed gradient; accumulator re-zeroed
//
// Main kernel.  A work item is one (batch, KV head, 128-key tile j); its CTA keeps K_j and V_j
// in shared memory and dK_j, dV_j in tensor memory while it walks over every query head of the
// group and every query tile i >= j.  Per (head, i), with everything transposed so that the
// 128 keys are the M dimension (TMEM lanes):
//     S^T  = K_j Q_i^T             SS-MMA  -> TMEM [0,128)
//     dP^T = V_j dO_i^T            SS-MMA  -> TMEM [128,256)
//     P^T  = exp2(S^T*c - lse2_q), dS^T = P^T o (dP^T - delta_q) * scale     softmax warps
//            both written as packed bf16 over the scores (each thread inside its own columns)
//            and dS^T also into shared memory (it is the M-major A operand of the dQ product)
//     dQ_i = dS K_j                SS-MMA  -> TMEM [128,256)  (dP^T is dead by then)
//     dV_j += P^T dO_i             TS-MMA  -> TMEM [384,512)
//     dK_j += dS^T Q_i             TS-MMA  -> TMEM [256,384)
// dQ_i is summed over key tiles by different CTAs: the tile leaves through shared memory (the
// dS^T buffer, free once the dQ product has read it) in four 128-row x 32-column chunks that
// TMA adds into the fp32 accumulator in L2 (cp.reduce.async.bulk), asynchronously to the
// threads; per-thread vector atomics proved several times slower.  The order of those
// additions is not fixed, so dQ is reproducible only up to fp32 summation order.
// Roles (384 threads): warp 0 = TMA producer, warp 1 = MMA issuer (one thread), warps 4..11 =
// softmax / dQ read-out / epilogue (two threads per key row, 64 query columns each; no
// exchange is needed because the backward has no row reductions).  Persistent, one CTA per
// SM, items dealt heaviest-first in zigzag order.  Every mbarrier wait is bounded.

#include <cstdint>
#include <cstdio>

#include "sm100_ptx.cuh"
#include "attention_sm100.h"

namespace elfb {

const char* make_tmap_2d(CUtensorMap* out, const void* ptr, int fmt, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                         uint32_t box_rows);
const char* make_tmap_out(CUtensorMap* out, const void* ptr, int fmt, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                          uint32_t box_rows);

namespace attn_bwd {

constexpr int D = 128;
constexpr int BT = 128;                 // keys per item, queries per iteration
constexpr int TILE_BYTES = 128 * D * 2;  // 32 KiB: two 64-column boxes of 128 rows
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int NUM_THREADS = 384;
constexpr int TMEM_COLS = 512;
constexpr int S_COL = 0, DP_COL = 128, DK_COL = 256, DV_COL = 384;
constexpr int STATS_BYTES = 2 * 2 * 128 * 4;  // [stage][lse2 | delta][query]
// K | V | Q[2] | dO[2] | dS | stats | barriers
constexpr size_t SMEM_BYTES = size_t(TILE_BYTES) * 7 + STATS_BYTES + 256;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct Item {
  int b, kv_head, j, n_iter;
};

struct ItemWalk {
  int n_tiles, n_kv_heads, group, per_level, total, cta, n_ctas;
  __device__ __forceinline__ bool get(int round, Item* it) const {
    const int idx = round * n_ctas + ((round & 1) ? (n_ctas - 1 - cta) : cta);
    if (idx >= total) return false;
    const int level = idx / per_level;  // key tile: the first ones see the most queries
    const int rem = idx - level * per_level;
    it->j = level;
    it->kv_head = rem % n_kv_heads;
    it->b = rem / n_kv_heads;
    it->n_iter = group * (n_tiles - level);
    return true;
  }
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmap_qkv, const __grid_constant__ CUtensorMap tmap_do, const __grid_constant__ CUtensorMap tmap_dq,
                const float* __restrict__ lse2,
                const float* __restrict__ delta, __nv_bfloat16* __restrict__ dqkv, float* __restrict__ dq_acc, int batch, int seq, int n_heads,
                int n_kv_heads, float scale, int* __restrict__ status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = smem_u32(smem_raw);
  if ((smem_base & 1023u) != 0) {  // the 128-byte swizzle needs 1024-byte aligned tiles
    if (threadIdx.x == 0 && status != nullptr && atomicCAS(status, kOk, kErrBadShape) == kOk) status[1] = 3900000;
    return;
  }
  const uint32_t k_smem = smem_base, v_smem = smem_base + TILE_BYTES;
  auto q_smem = [&](int s) { return smem_base + TILE_BYTES * (2 + s); };
  auto do_smem = [&](int s) { return smem_base + TILE_BYTES * (4 + s); };
  const uint32_t ds_smem = smem_base + TILE_BYTES * 6;
  float* stats = reinterpret_cast<float*>(smem_raw + size_t(TILE_BYTES) * 7);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + size_t(TILE_BYTES) * 7 + STATS_BYTES);
  const uint32_t bar0 = smem_u32(bars);
  enum { KV_FULL = 0, KV_EMPTY, Q_FULL, Q_EMPTY = Q_FULL + 2, SP_FULL = Q_EMPTY + 2, P_FULL, DQ_FULL, DQ_FREE, ACC_FULL, ACC_FREE, STG_FULL, STG_FREE = STG_FULL + 2, N_BARS = STG_FREE + 2 };
  auto bar = [&](int slot) { return bar0 + 8u * slot; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + N_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  ItemWalk walk;
  walk.n_tiles = seq / BT;
  walk.n_kv_heads = n_kv_heads;
  walk.group = n_heads / n_kv_heads;
  walk.per_level = batch * n_kv_heads;
  walk.total = walk.per_level * walk.n_tiles;
  walk.cta = blockIdx.x;
  walk.n_ctas = gridDim.x;
  const int pitch = (n_heads + 2 * n_kv_heads) * D;  // elements per token in the packed buffers
  const float scale_log2 = scale * 1.4426950408889634f;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar(KV_FULL), 1);
    mbar_init(bar(KV_EMPTY), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(Q_FULL + s), 1);
      mbar_init(bar(Q_EMPTY + s), 1);
    }
    mbar_init(bar(SP_FULL), 1);
    mbar_init(bar(P_FULL), 8);    // one arrival per softmax warp
    mbar_init(bar(DQ_FULL), 1);
    mbar_init(bar(DQ_FREE), 8);
    mbar_init(bar(ACC_FULL), 1);
    mbar_init(bar(ACC_FREE), 8);
    for (int h = 0; h < 2; ++h) {
      mbar_init(bar(STG_FULL + h), 4);  // the four warps of a column half have written their chunk
      mbar_init(bar(STG_FREE + h), 1);  // TMA has read it
    }
    fence_barrier_init();
    prefetch_tensormap(&tmap_qkv);
    prefetch_tensormap(&tmap_do);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // Iteration number `it` of an item -> (query head, query tile).  Query tiles run from the last
  // one down and the heads of the group are the inner loop, so that all CTAs sweep the query
  // range at the same pace: the rows of the fp32 dQ accumulator (and the Q / dO tiles) touched
  // at any moment are a window of a few megabytes that stays in L2, instead of the whole buffer.
  auto iter_coords = [&](const Item& item, int it, int* head, int* i) {
    const int step = it / walk.group;
    *head = item.kv_head * walk.group + (it - step * walk.group);
    *i = walk.n_tiles - 1 - step;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int qc = 0;  // iterations requested so far: stage qc & 1
      bool ok = true;
      Item item;
      for (int round = 0; ok && walk.get(round, &item); ++round) {
        // the previous item's last products have read K and V
        if (round > 0 && !mbar_wait(bar(KV_EMPTY), uint32_t(round - 1) & 1u, abort_flag)) break;
        const int key_row0 = item.b * seq + item.j * BT;
        const int k_col = (n_heads + item.kv_head) * D, v_col = (n_heads + n_kv_heads + item.kv_head) * D;
        mbar_arrive_expect_tx(bar(KV_FULL), 2 * TILE_BYTES);
        tma_load_2d(k_smem, &tmap_qkv, bar(KV_FULL), k_col, key_row0);
        tma_load_2d(k_smem + HALF_BYTES, &tmap_qkv, bar(KV_FULL), k_col + 64, key_row0);
        tma_load_2d(v_smem, &tmap_qkv, bar(KV_FULL), v_col, key_row0);
        tma_load_2d(v_smem + HALF_BYTES, &tmap_qkv, bar(KV_FULL), v_col + 64, key_row0);
        for (int it = 0; it < item.n_iter; ++it, ++qc) {
          const int stage = qc & 1;
          if (!mbar_wait(bar(Q_EMPTY + stage), (uint32_t(qc >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
          int head, i;
          iter_coords(item, it, &head, &i);
          const int q_row0 = item.b * seq + i * BT;
          const size_t stat_off = (size_t(item.b) * n_heads + head) * seq + size_t(i) * BT;
          const uint32_t fb = bar(Q_FULL + stage);
          mbar_arrive_expect_tx(fb, 2 * TILE_BYTES + 2 * 512);
          tma_load_2d(q_smem(stage), &tmap_qkv, fb, head * D, q_row0);
          tma_load_2d(q_smem(stage) + HALF_BYTES, &tmap_qkv, fb, head * D + 64, q_row0);
          tma_load_2d(do_smem(stage), &tmap_do, fb, head * D, q_row0);
          tma_load_2d(do_smem(stage) + HALF_BYTES, &tmap_do, fb, head * D + 64, q_row0);
          bulk_load_1d(smem_u32(stats + stage * 256), lse2 + stat_off, 512, fb);
          bulk_load_1d(smem_u32(stats + stage * 256 + 128), delta + stat_off, 512, fb);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_kk = make_idesc_f16(1u, BT, BT, 0u, 0u);  // S^T, dP^T: both operands K-major (contraction over d)
      const uint32_t idesc_mm = make_idesc_f16(1u, BT, D, 1u, 1u);   // dQ: A = dS (M-major), B = K (N-major), contraction over keys
      const uint32_t idesc_tm = make_idesc_f16(1u, BT, D, 0u, 1u);   // dV, dK: A from TMEM, B = dO / Q (N-major), contraction over queries
      int qc = 0;
      bool ok = true;
      Item item;
      for (int round = 0; ok && walk.get(round, &item); ++round) {
        if (!mbar_wait(bar(KV_FULL), uint32_t(round) & 1u, abort_flag)) break;
        for (int it = 0; it < item.n_iter; ++it, ++qc) {
          const int stage = qc & 1;
          if (!mbar_wait(bar(Q_FULL + stage), uint32_t(qc >> 1) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {  // S^T = K Q^T
            const uint32_t off = uint32_t(kk >> 2) * HALF_BYTES + uint32_t(kk & 3) * 32u;
            umma_ss(tmem_base + S_COL, make_smem_desc_sw128(k_smem + off, 0, 1024), make_smem_desc_sw128(q_smem(stage) + off, 0, 1024), idesc_kk, kk ? 1u : 0u);
          }
          // the previous iteration's dQ has been read out of the columns dP^T is about to overwrite
          if (qc > 0 && !mbar_wait(bar(DQ_FREE), uint32_t(qc - 1) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {  // dP^T = V dO^T
            const uint32_t off = uint32_t(kk >> 2) * HALF_BYTES + uint32_t(kk & 3) * 32u;
            umma_ss(tmem_base + DP_COL, make_smem_desc_sw128(v_smem + off, 0, 1024), make_smem_desc_sw128(do_smem(stage) + off, 0, 1024), idesc_kk, kk ? 1u : 0u);
          }
          umma_commit(bar(SP_FULL));
          if (!mbar_wait(bar(P_FULL), uint32_t(qc) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < BT / 16; ++kk) {  // dQ = dS K: 16 keys per step = 16 rows of 128 bytes in both tiles
            umma_ss(tmem_base + DP_COL, make_smem_desc_sw128(ds_smem + kk * 2048, HALF_BYTES, 1024), make_smem_desc_sw128(k_smem + kk * 2048, HALF_BYTES, 1024),
                    idesc_mm, kk ? 1u : 0u);
          }
          umma_commit(bar(DQ_FULL));
          // first products into dV / dK of this item: the previous item's epilogue has read them out
          if (it == 0 && round > 0 && !mbar_wait(bar(ACC_FREE), uint32_t(round - 1) & 1u, abort_flag)) { ok = false; break; }
#pragma unroll
          for (int kk = 0; kk < BT / 16; ++kk) {  // dV += P^T dO: 16 queries = 8 packed columns of P^T
            const uint32_t a = tmem_base + S_COL + (kk < 4 ? kk * 8 : 64 + (kk - 4) * 8);
            umma_ts(tmem_base + DV_COL, a, make_smem_desc_sw128(do_smem(stage) + kk * 2048, HALF_BYTES, 1024), idesc_tm, (it | kk) ? 1u : 0u);
          }
#pragma unroll
          for (int kk = 0; kk < BT / 16; ++kk) {  // dK += dS^T Q
            const uint32_t a = tmem_base + S_COL + 32 + (kk < 4 ? kk * 8 : 64 + (kk - 4) * 8);
            umma_ts(tmem_base + DK_COL, a, make_smem_desc_sw128(q_smem(stage) + kk * 2048, HALF_BYTES, 1024), idesc_tm, (it | kk) ? 1u : 0u);
          }
          umma_commit(bar(Q_EMPTY + stage));
        }
        if (!ok) break;
        umma_commit(bar(ACC_FULL));
        umma_commit(bar(KV_EMPTY));
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax, dQ read-out, epilogue
    const int quarter = warp & 3;        // TMEM lanes [32*quarter, +32)
    const int half = (warp - 4) >> 2;    // columns [64*half, +64) of every 128-column block
    const int r = quarter * 32 + lane;   // key row in the softmax and the epilogue, query row in the dQ read-out
    const uint32_t lane_off = uint32_t(quarter * 32) << 16;
    const uint32_t my_s = tmem_base + lane_off + S_COL + half * 64;  // this thread's 64 score columns; P^T -> first 32, dS^T -> last 32
    const uint32_t swz = uint32_t(r & 7);
    const uint32_t stg = ds_smem + uint32_t(half) * HALF_BYTES;  // this half's dS^T box doubles as its dQ staging chunk
    const bool stg_leader = (warp & 3) == 0 && lane == 0;          // one thread per half drives the TMA reductions
    int qc = 0;
    int cc = 0;  // dQ chunks this half has staged so far
    bool ok = true;
    Item item;
    for (int round = 0; ok && walk.get(round, &item); ++round) {
      for (int it = 0; it < item.n_iter; ++it, ++qc) {
        const int stage = qc & 1;
        int head, i;
        iter_coords(item, it, &head, &i);
        // lse2 / delta of this query tile arrived with the Q tile
        if (!mbar_wait(bar(Q_FULL + stage), uint32_t(qc >> 1) & 1u, abort_flag)) { ok = false; break; }
        if (!mbar_wait(bar(SP_FULL), uint32_t(qc) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const float4* lse_v = reinterpret_cast<const float4*>(stats + stage * 256 + half * 64);
        const float4* del_v = reinterpret_cast<const float4*>(stats + stage * 256 + 128 + half * 64);
        const bool diag = (i == item.j);
        // TMA has finished reading the previous iteration's last dQ chunk out of this half's dS^T box
        if (cc > 0 && !mbar_wait(bar(STG_FREE + half), uint32_t(cc - 1) & 1u, abort_flag)) { ok = false; break; }
        uint32_t s[2][32];
        tmem_ld_32x32b_x32(my_s, s[0]);
        tmem_ld_32x32b_x32(my_s + 32, s[1]);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t dp[32];
          tmem_ld_32x32b_x32(tmem_base + lane_off + DP_COL + half * 64 + c * 32, dp);
          tmem_ld_wait();  // covers the score loads too
          uint32_t pk[16], dk[16];
#pragma unroll
          for (int e4 = 0; e4 < 8; ++e4) {
            const float4 l4 = lse_v[c * 8 + e4];
            const float4 d4 = del_v[c * 8 + e4];
            const float lq[4] = {l4.x, l4.y, l4.z, l4.w};
            const float dq[4] = {d4.x, d4.y, d4.z, d4.w};
            float p[4], ds[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int col = c * 32 + e4 * 4 + e;  // query inside this thread's 64
              p[e] = fast_exp2(fmaf(__uint_as_float(s[c][e4 * 4 + e]), scale_log2, -lq[e]));
              if (diag && r > half * 64 + col) p[e] = 0.f;  // key after the query
              ds[e] = p[e] * (__uint_as_float(dp[e4 * 4 + e]) - dq[e]) * scale;
            }
            pk[e4 * 2] = pack_bf16x2(p[0], p[1]);
            pk[e4 * 2 + 1] = pack_bf16x2(p[2], p[3]);
            dk[e4 * 2] = pack_bf16x2(ds[0], ds[1]);
            dk[e4 * 2 + 1] = pack_bf16x2(ds[2], ds[3]);
          }
          tmem_st_32x32b_x16(my_s + c * 16, pk);        // P^T: queries 32c.. of this half -> packed columns 16c..
          tmem_st_32x32b_x16(my_s + 32 + c * 16, dk);   // dS^T
          // dS^T into shared memory as the M-major operand of dS K: box `half` holds queries 64*half.., one
          // 128-byte row per key, 16-byte chunks swizzled by the row
          const uint32_t row_base = ds_smem + uint32_t(half) * HALF_BYTES + uint32_t(r) * 128u;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint32_t dst = row_base + ((uint32_t(c * 4 + q) ^ swz) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(dk[4 * q]), "r"(dk[4 * q + 1]), "r"(dk[4 * q + 2]), "r"(dk[4 * q + 3]) : "memory");
          }
        }
        tmem_st_wait();
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(P_FULL));
        // ---- dQ read-out: lanes are query rows now; this thread adds d columns [64*half, +64) of its row
        if (!mbar_wait(bar(DQ_FULL), uint32_t(qc) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const int dq_row0 = item.b * seq + i * BT;
#pragma unroll 1
        for (int k = 0; k < 2; ++k, ++cc) {  // two 32-column chunks of this half's 64 columns
          uint32_t dq[32];
          tmem_ld_32x32b_x32(tmem_base + lane_off + DP_COL + half * 64 + k * 32, dq);
          tmem_ld_wait();
          if (k == 1) {
            // every dQ column of this thread has left tensor memory: dP^T of the next iteration may overwrite it
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(DQ_FREE));
          }
          // the staging chunk is free again once TMA has read the previous one
          if (cc > 0 && !mbar_wait(bar(STG_FREE + half), uint32_t(cc - 1) & 1u, abort_flag)) { ok = false; break; }
          const uint32_t row_base = stg + uint32_t(r) * 128u;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint32_t dst = row_base + ((uint32_t(q) ^ swz) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(dq[4 * q]), "r"(dq[4 * q + 1]), "r"(dq[4 * q + 2]), "r"(dq[4 * q + 3]) : "memory");
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(STG_FULL + half));
          if (stg_leader) {
            if (!mbar_wait(bar(STG_FULL + half), uint32_t(cc) & 1u, abort_flag)) { ok = false; }
            else {
              tma_reduce_add_2d(&tmap_dq, stg, head * D + half * 64 + k * 32, dq_row0);
              tma_store_commit();
              tma_store_wait_read<0>();
              mbar_arrive(bar(STG_FREE + half));
            }
          }
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;  // the leader's result reaches its warp
          if (!ok) break;
        }
        if (!ok) break;
      }
      if (!ok) break;
      // ---- epilogue of the item: dK_j, dV_j -> bf16 (each thread owns 128 bytes of a key row of each)
      if (!mbar_wait(bar(ACC_FULL), uint32_t(round) & 1u, abort_flag)) break;
      tc_fence_after_sync();
      const size_t token = size_t(item.b) * seq + size_t(item.j) * BT + r;
#pragma unroll
      for (int which = 0; which < 2; ++which) {  // 0: dK, 1: dV
        const uint32_t src = tmem_base + lane_off + (which ? DV_COL : DK_COL) + half * 64;
        const int col0 = (n_heads + (which ? n_kv_heads : 0) + item.kv_head) * D + half * 64;
        uint4* dst = reinterpret_cast<uint4*>(dqkv + token * pitch + col0);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(src + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[8 * q]), __uint_as_float(o[8 * q + 1]));
            w.y = pack_bf16x2(__uint_as_float(o[8 * q + 2]), __uint_as_float(o[8 * q + 3]));
            w.z = pack_bf16x2(__uint_as_float(o[8 * q + 4]), __uint_as_float(o[8 * q + 5]));
            w.w = pack_bf16x2(__uint_as_float(o[8 * q + 6]), __uint_as_float(o[8 * q + 7]));
            dst[c * 4 + q] = w;
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(ACC_FREE));
    }
    if (stg_leader) tma_store_wait_all();  // this thread's reductions have been performed
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
        status[1] = 3000000 + blockIdx.x;
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

// delta = rowsum(O o dO), lse2 = lse * log2(e).  One warp per (token, head) row of 128 elements.
__global__ void attn_bwd_prepare(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout, const float* __restrict__ lse,
                                 float* __restrict__ lse2, float* __restrict__ delta, int batch, int seq, int n_heads) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // token * n_heads + head
  const long long rows = (long long)batch * seq * n_heads;
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const uint2 a = reinterpret_cast<const uint2*>(out + row * D)[lane];
  const uint2 g = reinterpret_cast<const uint2*>(dout + row * D)[lane];
  const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
  float acc = 0.f;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const float2 x = __bfloat1622float2(a2[k]), y = __bfloat1622float2(g2[k]);
    acc += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) {
    const long long token = row / n_heads;
    const int head = int(row - token * n_heads);
    const long long b = token / seq, s = token - b * seq;
    const long long idx = (b * n_heads + head) * seq + s;
    delta[idx] = acc;
    lse2[idx] = lse[idx] * 1.4426950408889634f;
  }
}

// dQ accumulator (fp32 [tokens][Hq*128]) -> bf16 into the Q slots of the packed gradient; the accumulator is left zero.
__global__ void attn_bwd_finish(float* __restrict__ dq_acc, __nv_bfloat16* __restrict__ dqkv, long long tokens, int q_cols, int pitch) {
  const long long n4 = tokens * (q_cols / 4);
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n4; idx += (long long)gridDim.x * blockDim.x) {
    const long long token = idx / (q_cols / 4);
    const int c4 = int(idx - token * (q_cols / 4));
    float4* src = reinterpret_cast<float4*>(dq_acc) + idx;
    const float4 v = *src;
    *src = make_float4(0.f, 0.f, 0.f, 0.f);
    uint2 w;
    w.x = pack_bf16x2(v.x, v.y);
    w.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(dqkv + token * pitch + c4 * 4) = w;
  }
}

}  // namespace attn_bwd

const char* attention_backward(const AttnBwdArgs& a, cudaStream_t stream) {
  using namespace attn_bwd;
  if (a.batch <= 0 || a.seq <= 0) return nullptr;
  if (a.seq % BT != 0) return "attention: sequence length must be a multiple of 128";
  if (a.n_kv_heads <= 0 || a.n_heads % a.n_kv_heads != 0) return "attention: query heads must be a multiple of key/value heads";
  if ((reinterpret_cast<uintptr_t>(a.dqkv) & 15) != 0 || (reinterpret_cast<uintptr_t>(a.dq_acc) & 15) != 0 || (reinterpret_cast<uintptr_t>(a.lse2) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(a.delta) & 15) != 0 || (reinterpret_cast<uintptr_t>(a.out) & 7) != 0 || (reinterpret_cast<uintptr_t>(a.dout) & 15) != 0)
    return "attention: buffers must be 16-byte aligned";
  const uint64_t tokens = uint64_t(a.batch) * a.seq;
  const uint64_t pitch = uint64_t(a.n_heads + 2 * a.n_kv_heads) * D;
  const uint64_t q_cols = uint64_t(a.n_heads) * D;
  CUtensorMap tq, tdo, tdq;
  const char* err = make_tmap_2d(&tq, a.qkv, 1, tokens, pitch, pitch, 64, 128);
  if (err) return err;
  err = make_tmap_2d(&tdo, a.dout, 1, tokens, q_cols, q_cols, 64, 128);
  if (err) return err;
  err = make_tmap_out(&tdq, a.dq_acc, 2, tokens, q_cols, q_cols, 32, 128);  // fp32, 128-byte wide chunks
  if (err) return err;
  // SM count and function attributes are per device
  static int sms_of[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return "attention: cannot query the device";
  if (sms_of[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return "attention: cannot query the device";
    if (cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES) != cudaSuccess)
      return "attention: cannot raise the shared memory limit";
    sms_of[dev] = n;
  }
  const int num_sms = sms_of[dev];
  const float scale = a.scale > 0.f ? a.scale : 0.08838834764831845f;
  const long long rows = (long long)tokens * a.n_heads;
  attn_bwd_prepare<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(a.out), static_cast<const __nv_bfloat16*>(a.dout), a.lse, a.lse2,
                                                                   a.delta, a.batch, a.seq, a.n_heads);
  const long long items = (long long)(a.seq / BT) * a.n_kv_heads * a.batch;
  const int grid = int(items < num_sms ? items : num_sms);
  attn_bwd_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tq, tdo, tdq, a.lse2, a.delta, static_cast<__nv_bfloat16*>(a.dqkv), a.dq_acc, a.batch, a.seq, a.n_heads,
                                                             a.n_kv_heads, scale, a.status);
  attn_bwd_finish<<<num_sms * 8, 256, 0, stream>>>(a.dq_acc, static_cast<__nv_bfloat16*>(a.dqkv), (long long)tokens, (int)q_cols, (int)pitch);
  flush_bounds_record(a.status, stream);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace elfb
