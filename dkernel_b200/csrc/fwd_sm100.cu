// Prefill / training forward on the tcgen05 tensor cores (64-token blocks; head dim any multiple
// of 8 up to 256: the kernel is built for widths 64, 128 and 256, a narrower head is padded with
// the zeros TMA supplies for out-of-range columns, and only the real columns are stored).
//
// A 128-row query tile = two 64-row halves that share a kv head; S double buffered in TMEM,
// P overwrites S, O accumulates in TMEM; one converged issuer warp queues Q K_{j+2} right
// behind P V_j.  The CTAs are persistent: two per SM are launched and each walks a strided
// list of tiles, so that the per-tile fixed cost (block-list merge, pipeline fill, epilogue)
// overlaps the neighbouring tiles:
//   * a planner warp merges the next tile's block list while the current tile is computed
//     (two plan slots),
//   * the producer loads the next tile's Q as soon as the last Q K^T of the current tile has
//     completed, and its first K/V blocks as soon as their ring slots are free, i.e. while
//     the current tile's last softmax, P V and epilogue are still running,
//   * the issuer queues the next tile's first two Q K^T products right behind the last P V;
//     only the next tile's first P V (which overwrites O) waits for the epilogue.
// Block counters run across tiles, so buffer indices and barrier phases never restart.
// Warps (224 threads): 0-3 softmax + epilogue, 4 TMA producer, 5 MMA issuer (owns TMEM),
// 6 planner.  TMEM: S[2] 2x64 | O D columns.
// Math: dkernel/ops/sparse_attn_fwd.py:90-165, :351-363.
#include "ptx.cuh"

namespace bsa {
namespace {

constexpr int kBS = 64;
constexpr int kThreadsP = 224;
constexpr int kWarpProd = 4, kWarpIssue = 5, kWarpPlan = 6;
constexpr int kMaxList = 1024;           // kv blocks per sequence (64K tokens)
// Shared-memory tiles are stored as D/64 sub-tiles of [rows][128 bytes] (one TMA box each,
// 128-byte swizzled): Q 128 rows (16 KB per sub-tile), K and V 64 rows (8 KB per sub-tile).
template <int D> struct Geo {
  static constexpr int kSub = D / 64;
  static constexpr int kQBytes = 128 * D * 2;
  static constexpr int kTile = kBS * D * 2;           // one K or V block
  static constexpr size_t kSmem = 1024 + kQBytes + 2 * 2 * kTile;   // + sizeof(TailP)
};
constexpr float kRescaleThreshold = 8.0f;
enum { kPairHeads = 0, kPairRows = 1 };

struct Plan {
  int valid;                 // 0: nothing to do for this item (packed batches over-enumerate)
  int n;                     // number of kv blocks in list
  int b, kvh;
  int head[2], qblk[2], hvalid[2];
  int cbeg[2];               // first CSR entry of each half's pattern row (fine-block patterns)
  int q_start, q_len, k_start, k_len, past;
  uint16_t list[kMaxList];   // block | attended-by-half-0 << 14 | attended-by-half-1 << 15
};

struct TailP {
  uint64_t plan_full[2], plan_free[2];
  uint64_t q_full, q_free;
  uint64_t k_full[2], v_full[2];
  // qk_done[g&1]: Q K_g^T has completed -> S[g&1] is readable and the K slot is free.
  // pv_done[g&1]: P V_g has completed   -> the V slot is free (and O holds block g).
  uint64_t qk_done[2], p_full[2], pv_done[2];
  uint64_t o_free;           // the epilogue has read O
  uint32_t tmem_base;
  uint32_t bits[2][kMaxList / 32];
  Plan plan[2];
  // epilogue: 32 rows x 64 bytes per softmax warp, so that a store instruction covers whole
  // 64-byte row pieces of eight rows instead of 16 bytes of thirty-two rows
  alignas(16) uint8_t ostage[4][2048];
};


__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if (BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}

// item -> plan (executed by the whole planner warp)
__device__ __forceinline__ void build_plan(const bsa_fwd_params& p, int mode, int item, int tiles_x,
                                           int head_items, Plan* pl, uint32_t (*bits)[kMaxList / 32],
                                           int lane, int* wait_status) {
  const int tile_rows = mode == kPairHeads ? 64 : 128;
  // Items are ordered long rows first (the tile index decreases with the item index), all
  // heads and batches of a tile index together: a round of the grid then holds tiles of
  // nearly equal length, which keeps the CTAs' totals level.
  const int G = p.hq / p.hkv;
  const int per_tile = head_items * (p.total_q > 0 ? 1 : p.batch);
  const int tx = item / per_tile, rem = item % per_tile;
  const int hy = rem % head_items;
  int b = rem / head_items, tile = 0, valid = 1;
  if (p.total_q > 0) {
    int acc = 0;
    valid = 0;
    for (int i = 0; i < p.batch; ++i) {
      const int len = p.q_end[i] - p.q_start[i];
      const int nt = len > 0 ? (len + tile_rows - 1) / tile_rows : 0;
      if (tx < acc + nt) { b = i; tile = tx - acc; valid = 1; break; }
      acc += nt;
    }
  } else {
    tile = tiles_x - 1 - tx;
  }
  const int q_start = valid && p.q_start ? p.q_start[b] : 0;
  const int q_len = valid ? (p.q_end ? p.q_end[b] : p.sq) - q_start : 0;
  const int k_start = valid && p.k_start ? p.k_start[b] : 0;
  const int k_len = valid ? (p.k_end ? p.k_end[b] : p.sk) - k_start : 0;
  if (tile * tile_rows >= q_len) valid = 0;
  const int past = (p.causal || p.row_mode == BSA_ROWS_BY_POSITION) ? k_len - q_len : 0;
  int head[2], qblk[2], hvalid[2], kvh;
  if (mode == kPairHeads) {
    const int pairs = G / 2;
    kvh = hy / pairs;
    head[0] = kvh * G + 2 * (hy % pairs);
    head[1] = head[0] + 1;
    qblk[0] = qblk[1] = tile;
    hvalid[0] = hvalid[1] = valid;
  } else {
    head[0] = head[1] = hy;
    kvh = hy / G;
    qblk[0] = 2 * tile;
    qblk[1] = 2 * tile + 1;
    hvalid[0] = valid;
    hvalid[1] = valid && qblk[1] * kBS < q_len;
  }
  const int nkb = min((k_len + kBS - 1) / kBS, kMaxList);
  bits[0][lane] = 0u;
  bits[1][lane] = 0u;
  int cbeg[2] = {0, 0};
  __syncwarp();
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    if (!hvalid[t]) continue;
    const int q_first = qblk[t] * kBS;
    const int row = (p.row_mode == BSA_ROWS_BY_POSITION ? past + q_first : q_first) / kBS;
    if (row >= p.n_rows) continue;
    const int hp = pattern_head(head[t], p.h_pat, p.hq, p.hkv);
    const int32_t* cr = p.crow + (int64_t)hp * p.crow_sh;
    const int32_t* cols = p.col + (int64_t)hp * p.col_sh;
    const int c_beg = __ldg(cr + row), c_end = __ldg(cr + row + 1);
    cbeg[t] = c_beg;
    // a CSR row is a range of its head's column array
    if (!BSA_IN_BOUNDS(c_beg >= 0 && c_beg <= c_end && (p.col_sh == 0 || c_end <= p.col_sh), wait_status, 801))
      continue;
    const int q_pos_last = past + min(q_first + kBS, q_len) - 1;
    for (int i = c_beg + lane; i < c_end; i += 32) {
      const int blk = __ldg(cols + i);
      if (blk >= 0 && blk < nkb && !(p.causal && blk * kBS > q_pos_last))
        atomicOr(&bits[t][blk >> 5], 1u << (blk & 31));
    }
  }
  __syncwarp();
  // bitmaps -> ordered list: scan the word counts, then every lane owns one bit of a word
  const uint32_t u0 = bits[0][lane], u1 = bits[1][lane];
  const uint32_t u = u0 | u1;
  const int cnt = __popc(u);
  int incl = cnt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int tt = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += tt;
  }
  const int base = incl - cnt;
  uint32_t nonzero = __ballot_sync(0xffffffffu, u != 0u);
  while (nonzero) {
    const int w = __ffs(nonzero) - 1;
    nonzero &= nonzero - 1;
    const uint32_t uw = __shfl_sync(0xffffffffu, u, w);
    const uint32_t u0w = __shfl_sync(0xffffffffu, u0, w);
    const uint32_t u1w = __shfl_sync(0xffffffffu, u1, w);
    const int bw = __shfl_sync(0xffffffffu, base, w);
    if (((uw >> lane) & 1u) && BSA_IN_BOUNDS(bw + __popc(uw & ((1u << lane) - 1u)) < kMaxList, wait_status, 802))
      pl->list[bw + __popc(uw & ((1u << lane) - 1u))] =
          (uint16_t)((w * 32 + lane) | (((u0w >> lane) & 1u) << 14) | (((u1w >> lane) & 1u) << 15));
  }
  const int n = __shfl_sync(0xffffffffu, incl, 31);
  if (lane == 0) {
    pl->valid = valid;
    pl->n = valid ? n : 0;
    pl->b = b;
    pl->kvh = kvh;
    pl->head[0] = head[0]; pl->head[1] = head[1];
    pl->qblk[0] = qblk[0]; pl->qblk[1] = qblk[1];
    pl->hvalid[0] = hvalid[0]; pl->hvalid[1] = hvalid[1];
    pl->cbeg[0] = cbeg[0]; pl->cbeg[1] = cbeg[1];
    pl->q_start = q_start; pl->q_len = q_len; pl->k_start = k_start; pl->k_len = k_len;
    pl->past = past;
  }
  __syncwarp();
}

// FB: 0, or the pattern's own block size (16 or 32) when it is finer than the 64-token tiles: the
// CSR then describes the pattern coarsened to 64 x 64 blocks and col_bits holds, per CSR entry,
// one bit per (sub-row, sub-column) pair of the block (bit a * (64/FB) + b).
template <bool BF16, int D, int FB>
__global__ void __launch_bounds__(kThreadsP, D <= 128 ? 2 : 1)
fwd_persist_kernel(const __grid_constant__ Tmap4 tmQ, const __grid_constant__ Tmap4 tmK,
                   const __grid_constant__ Tmap4 tmV, bsa_fwd_params p, int mode, int n_items,
                   int tiles_x, int head_items, int* wait_status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  constexpr int kSub = Geo<D>::kSub, kQBytes = Geo<D>::kQBytes, kTile = Geo<D>::kTile;
  uint8_t* sQ = smem;                   // [kSub sub-tiles of 64 head dims][128 rows][128 B]
  uint8_t* sRing = smem + kQBytes;      // slot s: K at s * 2 * kTile, V one kTile behind it
  TailP* tl = reinterpret_cast<TailP*>(smem + kQBytes + 2 * 2 * kTile);

  if (*reinterpret_cast<volatile int*>(wait_status) != 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (warp == 0) {
    // seventeen contiguous barriers (plan_full[2], plan_free[2], q_full, q_free, k_full[2],
    // v_full[2], qk_done[2], p_full[2], pv_done[2], o_free); arrival counts: plan_free = 4
    // softmax warps + producer + issuer, p_full and o_free = 4 softmax warps, the rest 1
    if (lane < 17) {
      const int cnt = (lane == 2 || lane == 3) ? 6 : (lane == 12 || lane == 13 || lane == 16) ? 4 : 1;
      mbar_init(&tl->plan_full[0] + lane, cnt);
      mbar_fence_init();
    } else if (lane == 17) {
      tma_prefetch_desc(&tmQ.map);
    } else if (lane == 18) {
      tma_prefetch_desc(&tmK.map);
    } else if (lane == 19) {
      tma_prefetch_desc(&tmV.map);
    }
  }
  if (warp == kWarpIssue) {
    tmem_alloc(&tl->tmem_base, D <= 128 ? 256 : 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tl->tmem_base;
  const uint32_t tS[2] = {tmem, tmem + 64};
  const uint32_t tO = tmem + 128;

  if (warp == kWarpPlan) {
    // ============================================================ planner
    // The planner alone decides which items this CTA works on; the other warps follow the
    // plans until one is marked as the end (valid < 0).  With a tile counter the CTAs draw
    // items from it as they go (long tiles first, so the CTAs finish within one short tile of
    // each other); without one, round r hands items [r * grid, (r + 1) * grid) to the CTAs,
    // odd rounds in reverse CTA order so that no CTA collects the longest tile of every round.
    for (int k = 0;; ++k) {
      int item;
      if (p.tile_counter) {
        item = 0;
        if (lane == 0) item = atomicAdd(p.tile_counter, 1);
        item = __shfl_sync(0xffffffffu, item, 0);
      } else {
        const long long it = (long long)k * gridDim.x + ((k & 1) ? gridDim.x - 1 - blockIdx.x : blockIdx.x);
        item = it < n_items ? (int)it : n_items;
      }
      const int pb = k & 1;
      if (!mbar_wait(&tl->plan_free[pb], ((k >> 1) & 1) ^ 1, wait_status, 401)) break;
      if (item >= n_items || item < 0) {
        if (lane == 0) {
          tl->plan[pb].valid = -1;
          tl->plan[pb].n = 0;
          mbar_arrive(&tl->plan_full[pb]);
        }
        break;
      }
      build_plan(p, mode, item, tiles_x, head_items, &tl->plan[pb], tl->bits, lane, wait_status);
      if (lane == 0) mbar_arrive(&tl->plan_full[pb]);
    }
  } else if (warp == kWarpProd) {
    // ============================================================ TMA producer
    if (lane == 0) {
      uint32_t g = 0;      // kv blocks issued so far, over all tiles
      int k = 0, ko = 0;   // tiles seen / tiles with work
      bool ok = true;
      while (ok) {
        const int pb = k & 1;
        if (!mbar_wait(&tl->plan_full[pb], (k >> 1) & 1, wait_status, 402)) break;
        const Plan* pl = &tl->plan[pb];
        if (pl->valid < 0) break;
        const int n = pl->n;
        if (n > 0) {
          // the Q tile may be replaced once the previous tile's last Q K^T has completed
          if (ko > 0 && !mbar_wait(&tl->q_free, (ko - 1) & 1, wait_status, 403)) break;
          mbar_expect_tx(&tl->q_full, (uint32_t)(pl->hvalid[0] + pl->hvalid[1]) * (kQBytes / 2));
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (!pl->hvalid[t]) continue;
            // a tile of a valid half starts inside the stored rows of its head and batch entry
            (void)BSA_IN_BOUNDS(pl->q_start + pl->qblk[t] * kBS >= 0 && pl->q_start + pl->qblk[t] * kBS < p.sq &&
                                    pl->head[t] >= 0 && pl->head[t] < p.hq && pl->b >= 0 && pl->b < p.batch,
                                wait_status, 803);
            for (int c = 0; c < kSub; ++c)
              tma_load_tile(sQ + c * 16384 + t * 8192, &tmQ, &tl->q_full, c * 64,
                            pl->q_start + pl->qblk[t] * kBS, pl->head[t], pl->b);
          }
          ++ko;
          // K runs one block ahead of V: the slot of K_{g+1} is free once Q K_{g-1}^T has completed,
          // which is earlier than P V_{g-2} (the products run in the order P V_{g-3}, Q K_{g-1}^T,
          // P V_{g-2}); one thread waiting for the two in block order would hold K_{g+1} back by
          // most of a block period.
          auto load_k = [&](int j) -> bool {
            const uint32_t gk = g + (uint32_t)j;
            const int s = gk & 1;
            const int tok = pl->k_start + (int)(pl->list[j] & 0x3fffu) * kBS;
            uint8_t* kdst = sRing + s * 2 * kTile;
            // a listed block starts inside the stored keys of its kv head (its tail may be past them)
            (void)BSA_IN_BOUNDS(tok >= 0 && tok < p.sk && pl->kvh >= 0 && pl->kvh < p.hkv, wait_status, 804);
            if (!mbar_wait(&tl->qk_done[s], ((gk >> 1) & 1) ^ 1, wait_status, 404)) return false;
            mbar_expect_tx(&tl->k_full[s], kTile);
#pragma unroll
            for (int c = 0; c < kSub; ++c)
              tma_load_tile(kdst + c * 8192, &tmK, &tl->k_full[s], c * 64, tok, pl->kvh, pl->b);
            return true;
          };
          ok = load_k(0);
          for (int j = 0; j < n && ok; ++j) {
            if (j + 1 < n && !load_k(j + 1)) { ok = false; break; }
            const uint32_t gv = g + (uint32_t)j;
            const int s = gv & 1;
            const int tok = pl->k_start + (int)(pl->list[j] & 0x3fffu) * kBS;
            if (!mbar_wait(&tl->pv_done[s], ((gv >> 1) & 1) ^ 1, wait_status, 405)) { ok = false; break; }
            mbar_expect_tx(&tl->v_full[s], kTile);
#pragma unroll
            for (int c = 0; c < kSub; ++c)
              tma_load_tile(sRing + s * 2 * kTile + kTile + c * 8192, &tmV, &tl->v_full[s], c * 64, tok, pl->kvh,
                            pl->b);
          }
          g += (uint32_t)n;
        }
        if (ok) mbar_arrive(&tl->plan_free[pb]);
        ++k;
      }
    }
  } else if (warp == kWarpIssue) {
    // ============================================================ MMA issuer
    // The whole warp runs the loop converged, so that descriptors and addresses stay in
    // uniform registers; only the tcgen05 instructions sit under the elected lane.  Per
    // block the order is P V_g, Q K_{g+2}: the tensor pipe runs one thread's products in
    // issue order, so the product that overwrites P_g's columns needs no completion wait.
    const uint32_t idesc_qk = umma_idesc(BF16, 128, kBS, false, false);
    const uint32_t idesc_pv = umma_idesc(BF16, 128, D, false, true);
    const uint64_t qdesc0 = umma_desc_sw128(smem_u32(sQ), 16, 1024);
    const uint64_t kdesc0 = umma_desc_sw128(smem_u32(sRing), 16, 1024);
    // V tile read MN-major: 16 tokens (2 KB) per k-step, the two 64-dim halves 8 KB apart
    const uint64_t vdesc0 = umma_desc_sw128(smem_u32(sRing) + kTile, 8192, 1024);
    uint32_t g = 0;
    int k = 0, ko = 0;
    bool ok = true;
    // Q K^T of block gq (gq counts over all tiles); `last` marks the tile's last block
    auto issue_qk = [&](uint32_t gq, bool last) -> bool {
      const int s = gq & 1;
      if (!mbar_wait(&tl->k_full[s], (gq >> 1) & 1, wait_status, 411)) return false;
      tc_fence_after();
      const uint64_t db0 = kdesc0 + (uint64_t)((s * 2 * kTile) >> 4);
      if (elect_one()) {
#pragma unroll
        for (int i = 0; i < D / 16; ++i)   // i = c * 4 + kk: sub-tile c (8 KB apart for K, 16 KB for Q), k-step kk
          tc_mma_ss(tS[s], qdesc0 + (uint64_t)(((i >> 2) * 16384 + (i & 3) * 32) >> 4),
                    db0 + (uint64_t)(((i >> 2) * 8192 + (i & 3) * 32) >> 4), idesc_qk, i ? 1u : 0u);
        tc_commit(&tl->qk_done[s]);
        if (last) tc_commit(&tl->q_free);
      }
      __syncwarp();
      return true;
    };
    while (ok) {
      const int pb = k & 1;
      if (!mbar_wait(&tl->plan_full[pb], (k >> 1) & 1, wait_status, 412)) break;
      if (tl->plan[pb].valid < 0) break;
      const int n = tl->plan[pb].n;
      if (n > 0) {
        if (!mbar_wait(&tl->q_full, ko & 1, wait_status, 413)) break;
        for (int j = 0; j < 2 && j < n && ok; ++j) ok = issue_qk(g + j, j == n - 1);
        for (int j = 0; j < n && ok; ++j, ++g) {
          const int s = g & 1;
          // V first: its probe is then off the path between the softmax publishing P and P V
          if (!mbar_wait(&tl->v_full[s], (g >> 1) & 1, wait_status, 415)) { ok = false; break; }
          if (!mbar_wait(&tl->p_full[s], (g >> 1) & 1, wait_status, 414)) { ok = false; break; }
          // the previous tile's epilogue must have read O before it is overwritten
          if (j == 0 && ko > 0 && !mbar_wait(&tl->o_free, (ko - 1) & 1, wait_status, 416)) { ok = false; break; }
          tc_fence_after();
          const uint64_t dv0 = vdesc0 + (uint64_t)((s * 2 * kTile) >> 4);
          const uint32_t acc0 = j ? 1u : 0u;
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              tc_mma_ts(tO, tS[s] + kk * 8, dv0 + (uint64_t)((kk * 2048) >> 4), idesc_pv, kk ? 1u : acc0);
            tc_commit(&tl->pv_done[s]);
          }
          __syncwarp();
          if (j + 2 < n) ok = issue_qk(g + 2, j + 2 == n - 1);
        }
        ++ko;
      }
      if (ok && elect_one()) mbar_arrive(&tl->plan_free[pb]);
      __syncwarp();
      ++k;
    }
  } else if (warp < 4) {
    // ============================================================ softmax + epilogue (warps 0-3)
    const int r = tid;            // tile row = TMEM lane
    const int t = r >> 6;         // half
    const int rr = r & 63;
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
    const float scale2 = p.sm_scale * kLog2e;
    const bool wide = reinterpret_cast<uintptr_t>(p.o) % 16 == 0 && p.o_ss % 8 == 0 &&
                      p.o_sh % 8 == 0 && p.o_sb % 8 == 0;   // rows start on 16-byte boundaries
    uint32_t g = 0;      // kv blocks processed so far, over all tiles
    // Completion of P V_x.  A parity wait is unambiguous while the barrier can be at most one
    // phase past the awaited one: that holds for x = g-1 while block g is being processed (the
    // barrier's next phase, P V_{g+1}, needs this warp's P_{g+1}) and for the last block of a
    // tile in its epilogue.  P V_{g-2} needs no wait at all: Q K_g^T was queued behind it and
    // the tensor pipe runs in order, so S_g being readable implies it has completed.
    auto wait_pv = [&](uint32_t x) {
      return mbar_wait(&tl->pv_done[x & 1], (x >> 1) & 1, wait_status, 421);
    };
    int k = 0;
    bool alive = true;
    while (alive) {
      const int pb = k & 1;
      if (!mbar_wait(&tl->plan_full[pb], (k >> 1) & 1, wait_status, 422)) break;
      const Plan* pl = &tl->plan[pb];
      if (pl->valid < 0) break;
      const int n = pl->n;
      const int hvalid = pl->hvalid[t], head = pl->head[t];
      const int q_row = pl->qblk[t] * kBS + rr;   // row inside the sequence
      const int q_len = pl->q_len, k_len = pl->k_len, b = pl->b;
      const int qpos = pl->past + q_row;
      const bool row_ok = hvalid && q_row < q_len;
      uint8_t* orow = reinterpret_cast<uint8_t*>(p.o) +
                      ((int64_t)b * p.o_sb + (int64_t)head * p.o_sh + (int64_t)(pl->q_start + q_row) * p.o_ss) * 2;
      float* lse_ptr = p.lse ? p.lse + (int64_t)b * p.lse_sb + (int64_t)head * p.lse_sh + pl->q_start + q_row
                             : nullptr;
      if (n == 0) {
        if (pl->valid && row_ok) {   // a tile that attends nothing: zero rows, LSE = -inf
          for (int i = 0; i < p.d / 4; ++i) reinterpret_cast<uint2*>(orow)[i] = make_uint2(0u, 0u);
          if (lse_ptr) *lse_ptr = -INFINITY;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&tl->plan_free[pb]);
        ++k;
        continue;
      }
      float m_used = -INFINITY, l = 0.f;
      // fine-block patterns: this half's entries of the tile are a prefix of its CSR row, in order
      constexpr int kF = FB ? kBS / FB : 1;                  // sub-blocks per side
      constexpr uint32_t kFull = (1u << kF) - 1u;
      const int32_t* fbits = nullptr;
      if (FB) {
        const int hp = pattern_head(head, p.h_pat, p.hq, p.hkv);
        fbits = p.col_bits + (int64_t)hp * p.col_bits_sh + pl->cbeg[t];
      }
      for (int j = 0; j < n; ++j, ++g) {
        const int s = g & 1;
        // everything that only depends on the block list is done before the barrier probe
        const uint32_t ent = pl->list[j];
        const int kbase = (int)(ent & 0x3fffu) * kBS;
        const bool att = ((ent >> (14 + t)) & 1u) != 0 && hvalid;
        int lim = k_len - kbase;
        if (p.causal) lim = min(lim, qpos - kbase + 1);
        uint32_t cm = kFull;     // which sub-columns this row attends inside the block
        if (FB && att) cm = ((uint32_t)__ldg(fbits++) >> ((rr / (FB ? FB : 1)) * kF)) & kFull;
        // the entries of this half that the tile walks are a prefix of its CSR row
        if (FB && att)
          (void)BSA_IN_BOUNDS(p.col_bits_sh == 0 || fbits - p.col_bits - (int64_t)pattern_head(head, p.h_pat, p.hq, p.hkv) *
                                                                         p.col_bits_sh <= p.col_bits_sh,
                              wait_status, 806);
        if (!mbar_wait(&tl->qk_done[s], (g >> 1) & 1, wait_status, 423)) { alive = false; break; }
        tc_fence_after();
        uint32_t sv[64];
        tmem_ld32(tS[s] + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
        tmem_ld32(tS[s] + lane_off + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
        tmem_ld_wait();
        // Allowed columns of this block form a prefix: kpos < k_len and, when causal,
        // kpos <= qpos.  Raw logits are compared (sm_scale > 0); the scale is folded
        // into the exponent's FMA.
        float mx = -INFINITY;
        if (att) {
          if (lim < kBS) {
#pragma unroll
            for (int c = 0; c < 64; ++c)
              if (c >= lim) sv[c] = 0xff800000u;  // -inf
          }
          if (FB && cm != kFull) {
#pragma unroll
            for (int c = 0; c < 64; ++c)
              if (!((cm >> (c / (FB ? FB : 1))) & 1u)) sv[c] = 0xff800000u;
          }
          float m4[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) m4[i] = max3(__uint_as_float(sv[3 * i]), __uint_as_float(sv[3 * i + 1]),
                                                   __uint_as_float(sv[3 * i + 2]));
#pragma unroll
          for (int c = 12; c < 60; c += 8)
#pragma unroll
            for (int i = 0; i < 4; ++i)
              m4[i] = max3(m4[i], __uint_as_float(sv[c + 2 * i]), __uint_as_float(sv[c + 2 * i + 1]));
          mx = max3(max3(m4[0], m4[1], m4[2]), max3(m4[3], __uint_as_float(sv[60]), __uint_as_float(sv[61])),
                    fmaxf(__uint_as_float(sv[62]), __uint_as_float(sv[63]))) * scale2;
        }
        float alpha = 1.f;
        bool need = false;
        if (att && mx != -INFINITY) {
          if (m_used == -INFINITY) {
            m_used = mx;   // first attended block of this row: its O row is still exactly 0
          } else if (mx > m_used + kRescaleThreshold) {
            alpha = ex2(m_used - mx);
            m_used = mx;
            l *= alpha;
            need = true;
          }
        }
        const bool any = __any_sync(0xffffffffu, need);
        // P is produced and stored in two halves, so that the first store's latency is covered
        // by the second half's exponentials and fewer packed values are live at a time
        const bool live = att && m_used != -INFINITY;
        const float neg_m = -m_used;
        // two columns per fused multiply-add and per addition (packed fp32 pairs): the softmax
        // warps are bound by instruction issue as much as by the exponential unit
        const uint64_t scale_2 = f32x2(scale2, scale2), neg_m2 = f32x2(neg_m, neg_m);
        uint64_t sum2[2] = {0ull, 0ull};
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
          uint32_t pk[16];
          if (live) {
#pragma unroll
            for (int c = 0; c < 16; ++c) {
              float x0, x1;
              f32x2_split(fma_f32x2(f32x2(sv[hlf * 32 + 2 * c], sv[hlf * 32 + 2 * c + 1]), scale_2, neg_m2), x0, x1);
              const float p0 = ex2(x0), p1 = ex2(x1);
              sum2[c & 1] = add_f32x2(sum2[c & 1], f32x2(p0, p1));
              pk[c] = pack2<BF16>(p0, p1);
            }
          } else {
#pragma unroll
            for (int c = 0; c < 16; ++c) pk[c] = 0u;
          }
          tmem_st16(tS[s] + lane_off + hlf * 16, pk);
        }
        float sum[4];
        f32x2_split(sum2[0], sum[0], sum[1]);
        f32x2_split(sum2[1], sum[2], sum[3]);
        l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
        if (any && j > 0) {
          // rescale the accumulator rows whose maximum moved, once P V_{g-1} has landed
          if (!wait_pv(g - 1)) { alive = false; break; }
          tc_fence_after();
#pragma unroll
          for (int ch = 0; ch < D / 32; ++ch) {
            uint32_t o[32];
            tmem_ld32(tO + lane_off + ch * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(tO + lane_off + ch * 32, o);
          }
        }
        if (k_len - kbase < kBS) {
          // The block reaches past the end of the sequence.  Its logits are masked above, but the
          // P V product still reads the whole V tile, and rows past the end hold whatever the
          // caller's buffer holds there (0 * NaN = NaN): clear them in shared memory.
          if (!mbar_wait(&tl->v_full[s], (g >> 1) & 1, wait_status, 424)) { alive = false; break; }
          uint8_t* vt = sRing + s * 2 * kTile + kTile;
          const int first = k_len - kbase;   // >= 1: blocks that start at or past the end are not listed
          for (int idx = tid; idx < (kBS - first) * kSub * 8; idx += 128) {
            const int row = first + idx / (kSub * 8), c = (idx / 8) % kSub, ch = idx & 7;
            *reinterpret_cast<uint4*>(vt + c * 8192 + row * 128 + ch * 16) = make_uint4(0u, 0u, 0u, 0u);
          }
          fence_proxy_async();   // generic-proxy writes -> visible to the tensor core's reads
        }
        // tcgen05.wait::st is warp-wide: after it every lane's P row is in TMEM, so one
        // arrival per warp publishes them
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tl->p_full[s]);
      }
      if (!alive) break;
      // ---- epilogue of the tile: all its P V products must have completed; each thread
      // normalises its own row and stores it straight from registers
      if (!wait_pv(g - 1)) { alive = false; break; }
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
      for (int ch = 0; ch < D / 32; ++ch) {
        uint32_t o[32];
        tmem_ld32(tO + lane_off + ch * 32, o);
        tmem_ld_wait();
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
          w[i] = pack2<BF16>(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
        if (ch == D / 32 - 1) {
          // O has been read: the next tile's first P V may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tl->o_free);
        }
        if (wide) {
          // own row -> staging (16-byte pieces, swizzled by the row pair: conflict-free both ways),
          // then lane L stores piece L % 4 of rows L / 4, L / 4 + 8, ...
          uint8_t* stg = tl->ostage[warp];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            *reinterpret_cast<uint4*>(stg + lane * 64 + ((i ^ ((lane >> 1) & 3)) * 16)) =
                make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
          __syncwarp();
          const int pc = lane & 3;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int sr = i * 8 + (lane >> 2);            // row of this warp's 32
            const uint4 val = *reinterpret_cast<const uint4*>(stg + sr * 64 + ((pc ^ ((sr >> 1) & 3)) * 16));
            const int srow = q_row - lane + sr;            // row inside the sequence
            if (hvalid && srow < q_len && ch * 32 + pc * 8 < p.d &&   // columns past the real head dim are padding
                BSA_IN_BOUNDS(pl->q_start + srow >= 0 && pl->q_start + srow < p.sq, wait_status, 805))
              *reinterpret_cast<uint4*>(orow + (int64_t)(sr - lane) * p.o_ss * 2 + ch * 64 + pc * 16) = val;
          }
          __syncwarp();   // the next chunk overwrites the staging rows
        } else if (row_ok && BSA_IN_BOUNDS(pl->q_start + q_row >= 0 && pl->q_start + q_row < p.sq, wait_status, 805)) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (ch * 32 + i * 4 < p.d)
              *reinterpret_cast<uint2*>(orow + ch * 64 + i * 8) = make_uint2(w[2 * i], w[2 * i + 1]);
        }
      }
      if (row_ok && lse_ptr) *lse_ptr = l > 0.f ? (m_used + log2f(l)) * kLn2 : -INFINITY;
      __syncwarp();
      if (lane == 0) mbar_arrive(&tl->plan_free[pb]);
      ++k;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kWarpIssue) tmem_dealloc(tmem, D <= 128 ? 256 : 512);
}

}  // namespace

bool sm100_fwd_supported(const bsa_fwd_params* p, const char** why) {
  auto no = [&](const char* w) { *why = w; return false; };
  if (!(p->dtype == BSA_F16 || p->dtype == BSA_BF16)) return no("dtype is not f16/bf16");
  if (p->d < 16 || p->d > 256 || p->d % 8) return no("head dim is not a multiple of 8 in [16, 256]");
  if (p->block_size != kBS) return no("block size is not 64");
  if (p->fine_block != 0) {
    if (p->fine_block != 16 && p->fine_block != 32) return no("fine_block is not 16 or 32");
    if (!p->col_bits) return no("fine_block without col_bits");
    if (p->d > 128) return no("fine-block patterns are served for head dims up to 128");
  }
  if (p->sk > kMaxList * kBS) return no("more than 65536 key positions");
  if (!tma_compatible(p->q, 2, p->q_ss, p->q_sh, p->q_sb) ||
      !tma_compatible(p->k, 2, p->k_ss, p->k_sh, p->k_sb) ||
      !tma_compatible(p->v, 2, p->v_ss, p->v_sh, p->v_sb))
    return no("q/k/v need 16-byte aligned bases and strides that are multiples of 16 bytes");
  if (reinterpret_cast<uintptr_t>(p->o) % 8 || p->o_ss % 4 || p->o_sh % 4 || p->o_sb % 4)
    return no("output rows are not 8-byte aligned");
  if (p->sq == 0 || p->batch == 0) return no("empty problem");
  if (!(p->sm_scale > 0.f)) return no("sm_scale is not positive");
  return true;
}

namespace {
template <bool BF16, int D, int FB>
int launch_fwd(const bsa_fwd_params* p, cudaStream_t s) {
  Tmap4 tmQ, tmK, tmV;
  const uint64_t nb = p->total_q > 0 ? 1 : p->batch;
  int rc = make_tmap_4d(&tmQ, p->q, 2, p->d, p->sq, p->hq, nb, p->q_ss * 2, p->q_sh * 2, p->q_sb * 2, 64, 64,
                        true, BF16);
  if (rc) return rc;
  rc = make_tmap_4d(&tmK, p->k, 2, p->d, p->sk, p->hkv, nb, p->k_ss * 2, p->k_sh * 2, p->k_sb * 2, 64, 64,
                    true, BF16);
  if (rc) return rc;
  rc = make_tmap_4d(&tmV, p->v, 2, p->d, p->sk, p->hkv, nb, p->v_ss * 2, p->v_sh * 2, p->v_sb * 2, 64, 64,
                    true, BF16);
  if (rc) return rc;
  const int G = p->hq / p->hkv;
  // Two heads share a tile only when they share a block list (one pattern for all heads
  // or one per kv head): with per-head patterns the union of two heads' lists would spend
  // half of the tensor work of every unshared block on an unattended half.  Two adjacent
  // row blocks of one head share all but the two ends of their lists.
  const int mode = (G % 2 == 0 && p->h_pat != p->hq) ? kPairHeads : kPairRows;
  const int tile_rows = mode == kPairHeads ? 64 : 128;
  const int head_items = mode == kPairHeads ? p->hq / 2 : p->hq;
  const int tiles_x = p->total_q > 0 ? cdiv_i(p->total_q, tile_rows) + p->batch : cdiv_i(p->sq, tile_rows);
  const long long n_items_ll = (long long)tiles_x * head_items * (p->total_q > 0 ? 1 : p->batch);
  if (n_items_ll > 0x7fffffffLL) {
    set_error("bsa_fwd: too many tiles for one launch");
    return BSA_E_TOOBIG;
  }
  const int n_items = (int)n_items_ll;
  int dev = 0, sms = 148;
  BSA_CHECK_CUDA(cudaGetDevice(&dev));
  BSA_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int per_sm = D <= 128 ? 2 : 1;                       // resident CTAs per SM (TMEM, shared memory)
  const int grid = n_items < per_sm * sms ? n_items : per_sm * sms;
  int* status = wait_status_ptr();
  if (!status) return BSA_E_CUDA;
  constexpr size_t smem = Geo<D>::kSmem + sizeof(TailP);
  auto kern = fwd_persist_kernel<BF16, D, FB>;
  BSA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<grid, kThreadsP, smem, s>>>(tmQ, tmK, tmV, *p, mode, n_items, tiles_x, head_items, status);
  return check_launch("fwd_persist_kernel");
}
}  // namespace

int sm100_fwd(const bsa_fwd_params* p, cudaStream_t s) {
  const bool bf16 = p->dtype == BSA_BF16;
  if (p->fine_block == 16) {
    if (p->d <= 64) return bf16 ? launch_fwd<true, 64, 16>(p, s) : launch_fwd<false, 64, 16>(p, s);
    return bf16 ? launch_fwd<true, 128, 16>(p, s) : launch_fwd<false, 128, 16>(p, s);
  }
  if (p->fine_block == 32) {
    if (p->d <= 64) return bf16 ? launch_fwd<true, 64, 32>(p, s) : launch_fwd<false, 64, 32>(p, s);
    return bf16 ? launch_fwd<true, 128, 32>(p, s) : launch_fwd<false, 128, 32>(p, s);
  }
  if (p->d <= 64) return bf16 ? launch_fwd<true, 64, 0>(p, s) : launch_fwd<false, 64, 0>(p, s);
  if (p->d <= 128) return bf16 ? launch_fwd<true, 128, 0>(p, s) : launch_fwd<false, 128, 0>(p, s);
  return bf16 ? launch_fwd<true, 256, 0>(p, s) : launch_fwd<false, 256, 0>(p, s);
}

}  // namespace bsa
