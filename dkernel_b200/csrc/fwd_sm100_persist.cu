// Prefill / training forward, persistent version with the Q tile resident in TMEM.
//
// Same tiling as the first tcgen05 forward (a 128-row query tile = two 64-row
// halves that share a kv head, union of the halves' CSR rows), but organised around
// what the profiles of that kernel showed:
//   * SS-mode Q K^T re-reads the 32 KB Q tile from shared memory for every kv block,
//     and the shared-memory read path (128 B/clk) was the busiest unit.  Here Q is
//     copied once per tile into TMEM (tcgen05.cp, 64 columns) and Q K^T runs in TS
//     mode, so a kv block costs 16 KB (K) + 16 KB (V) of operand reads.
//   * a third of the run time was per-CTA fixed cost (barrier set-up, list merge,
//     TMEM allocation, first loads, epilogue).  Here one CTA per SM is launched and
//     loops over tiles; a planner/producer warp merges the next tile's block list and
//     prefetches its Q tile and first K/V blocks while the current tile is computed.
//   * one hand-off between roles costs a few hundred cycles; S is triple buffered in
//     TMEM and the K/V ring is four blocks deep so that no role waits on another in
//     steady state.
// TMEM (512 columns): Q[2] 2x64 | S[3] 3x64 (P overwrites S) | O 128.
// Warps: 0-7 softmax (lane quadrant x 32-column half; the two warps of a row pair
// exchange their partial row maxima through shared memory), 8 planner + TMA
// producer, 9 Q-copy + Q K^T issuer (owns TMEM), 10 P V issuer.
// Math: dkernel/ops/sparse_attn_fwd.py:90-165, :351-363.
#include "ptx.cuh"

namespace bsa {
namespace {

constexpr int kD = 128;
constexpr int kBS = 64;
constexpr int kThreadsP = 352;
constexpr int kWarpProd = 8, kWarpA = 9, kWarpB = 10;
constexpr int kMaxList = 1024;           // kv blocks per sequence (64K tokens)
constexpr int kQBytes = 128 * kD * 2;    // 32 KB
constexpr int kTile = kBS * kD * 2;      // 16 KB: one K or V block
constexpr int kRing = 4;                 // K/V ring depth
constexpr int kSBuf = 3;                 // S/P buffers in TMEM
constexpr float kRescaleThreshold = 8.0f;
enum { kPairHeads = 0, kPairRows = 1 };

struct Plan {
  int valid;                 // 0: nothing to do for this item (packed batches over-enumerate)
  int n;                     // number of kv blocks in list
  int b, kvh;
  int head[2], qblk[2], hvalid[2];
  int q_start, q_len, k_start, k_len, past;
  uint16_t list[kMaxList];   // block | attended-by-half-0 << 14 | attended-by-half-1 << 15
};

struct TailP {
  uint64_t plan_full[2], plan_free[2];
  uint64_t q_full[2], q_stage_free[2];
  uint64_t k_full[kRing], v_full[kRing], k_free[kRing], v_free[kRing];
  uint64_t qk_done[kSBuf], p_full[kSBuf], pv_done[kSBuf];
  uint64_t o_free;
  uint32_t tmem_base;
  uint32_t bits[2][kMaxList / 32];
  float xch[2][2][128];      // [iteration parity][column half][row]: partial row maxima / sums
  Plan plan[2];
};

constexpr size_t kSmemP = 1024 + 2 * kQBytes + kRing * 2 * kTile + sizeof(TailP);

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
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
// first TMEM column of the packed P values of k-step kk (see the softmax role)
__device__ __forceinline__ uint32_t packed_col(int kk) { return (uint32_t)((kk >> 1) * 32 + (kk & 1) * 8); }
__device__ __forceinline__ void pair_bar(int quad) {
  asm volatile("bar.sync %0, 64;" ::"r"(quad + 1) : "memory");
}

// item -> plan (executed by the whole producer warp)
__device__ __forceinline__ void build_plan(const bsa_fwd_params& p, int mode, int item, int tiles_x,
                                           int head_items, Plan* pl, uint32_t (*bits)[kMaxList / 32],
                                           int lane) {
  const int G = p.hq / p.hkv;
  const int tile_rows = mode == kPairHeads ? 64 : 128;
  // items are ordered long rows first: the tile index decreases with the item index
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
  __syncwarp();
  for (int t = 0; t < 2; ++t) {
    if (!hvalid[t]) continue;
    const int q_first = qblk[t] * kBS;
    const int row = (p.row_mode == BSA_ROWS_BY_POSITION ? past + q_first : q_first) / kBS;
    if (row >= p.n_rows) continue;
    const int hp = pattern_head(head[t], p.h_pat, p.hq, p.hkv);
    const int32_t* cr = p.crow + (int64_t)hp * p.crow_sh;
    const int32_t* cols = p.col + (int64_t)hp * p.col_sh;
    const int c_beg = cr[row], c_end = cr[row + 1];
    const int q_pos_last = past + min(q_first + kBS, q_len) - 1;
    for (int i = c_beg + lane; i < c_end; i += 32) {
      const int blk = cols[i];
      if (blk >= 0 && blk < nkb && !(p.causal && blk * kBS > q_pos_last))
        atomicOr(&bits[t][blk >> 5], 1u << (blk & 31));
    }
  }
  __syncwarp();
  const uint32_t u0 = bits[0][lane], u1 = bits[1][lane];
  uint32_t u = u0 | u1;
  const int cnt = __popc(u);
  int incl = cnt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int tt = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += tt;
  }
  int pos = incl - cnt;
  while (u) {
    const int bit = __ffs(u) - 1;
    u &= u - 1;
    pl->list[pos++] = (uint16_t)((lane * 32 + bit) | (((u0 >> bit) & 1u) << 14) | (((u1 >> bit) & 1u) << 15));
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
    pl->q_start = q_start; pl->q_len = q_len; pl->k_start = k_start; pl->k_len = k_len;
    pl->past = past;
  }
  __syncwarp();
}

template <bool BF16>
__global__ void __launch_bounds__(kThreadsP, 1)
fwd_persist_kernel(const __grid_constant__ Tmap4 tmQ, const __grid_constant__ Tmap4 tmK,
                   const __grid_constant__ Tmap4 tmV, bsa_fwd_params p, int mode, int n_items,
                   int tiles_x, int head_items, int* wait_status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sQ = smem;                       // two staging tiles, 32 KB each
  uint8_t* sRing = smem + 2 * kQBytes;      // stage s: K at s*32K, V at s*32K + 16K
  TailP* tl = reinterpret_cast<TailP*>(smem + 2 * kQBytes + kRing * 2 * kTile);

  if (*reinterpret_cast<volatile int*>(wait_status) != 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tl->plan_full[i], 1);
      mbar_init(&tl->plan_free[i], 258);
      mbar_init(&tl->q_full[i], 1);
      mbar_init(&tl->q_stage_free[i], 1);
    }
    for (int i = 0; i < kRing; ++i) {
      mbar_init(&tl->k_full[i], 1);
      mbar_init(&tl->v_full[i], 1);
      mbar_init(&tl->k_free[i], 1);
      mbar_init(&tl->v_free[i], 1);
    }
    for (int i = 0; i < kSBuf; ++i) {
      mbar_init(&tl->qk_done[i], 1);
      mbar_init(&tl->p_full[i], 256);
      mbar_init(&tl->pv_done[i], 1);
    }
    mbar_init(&tl->o_free, 256);
    mbar_fence_init();
    tma_prefetch_desc(&tmQ.map);
    tma_prefetch_desc(&tmK.map);
    tma_prefetch_desc(&tmV.map);
  }
  if (warp == kWarpA) {
    tmem_alloc(&tl->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tl->tmem_base;
  const uint32_t tQ[2] = {tmem, tmem + 64};
  const uint32_t tS0 = tmem + 128;          // S buffer i at tS0 + 64 i
  const uint32_t tO = tmem + 320;

  if (warp == kWarpProd) {
    // ============================================================ planner + TMA producer
    uint32_t g = 0;
    int k = 0, ko = 0;   // items seen / items with work (the Q buffers cycle with the latter)
    for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++k) {
      const int pb = k & 1;
      if (!mbar_wait(&tl->plan_free[pb], ((k >> 1) & 1) ^ 1, wait_status, 401)) break;
      Plan* pl = &tl->plan[pb];
      build_plan(p, mode, item, tiles_x, head_items, pl, tl->bits, lane);
      const int n = pl->n;
      if (lane == 0) {
        mbar_arrive(&tl->plan_full[pb]);
        if (n > 0) {
          const int qb = ko & 1;
          bool ok = mbar_wait(&tl->q_stage_free[qb], ((ko >> 1) & 1) ^ 1, wait_status, 402);
          if (ok) {
            mbar_expect_tx(&tl->q_full[qb], (uint32_t)(pl->hvalid[0] + pl->hvalid[1]) * (kQBytes / 2));
            for (int t = 0; t < 2; ++t) {
              if (!pl->hvalid[t]) continue;
              for (int c = 0; c < 2; ++c)
                tma_load_tile(sQ + qb * kQBytes + c * 16384 + t * 8192, &tmQ, &tl->q_full[qb], c * 64,
                              pl->q_start + pl->qblk[t] * kBS, pl->head[t], pl->b);
            }
          }
          for (int j = 0; j < n && ok; ++j, ++g) {
            const int st = g % kRing;
            const uint32_t ph = ((g / kRing) & 1) ^ 1;
            const int tok = pl->k_start + (int)(pl->list[j] & 0x3fffu) * kBS;
            uint8_t* kdst = sRing + st * 2 * kTile;
            if (!mbar_wait(&tl->k_free[st], ph, wait_status, 403)) { ok = false; break; }
            mbar_expect_tx(&tl->k_full[st], kTile);
            tma_load_tile(kdst, &tmK, &tl->k_full[st], 0, tok, pl->kvh, pl->b);
            tma_load_tile(kdst + 8192, &tmK, &tl->k_full[st], 64, tok, pl->kvh, pl->b);
            if (!mbar_wait(&tl->v_free[st], ph, wait_status, 404)) { ok = false; break; }
            mbar_expect_tx(&tl->v_full[st], kTile);
            tma_load_tile(kdst + kTile, &tmV, &tl->v_full[st], 0, tok, pl->kvh, pl->b);
            tma_load_tile(kdst + kTile + 8192, &tmV, &tl->v_full[st], 64, tok, pl->kvh, pl->b);
          }
        }
      }
      if (n > 0) ++ko;
      // every lane needs the advanced block counter and the go/no-go decision
      g = __shfl_sync(0xffffffffu, g, 0);
      if (*reinterpret_cast<volatile int*>(wait_status) != 0) break;
    }
  } else if (warp == kWarpA) {
    // ============================================================ Q copy + Q K^T issuer
    if (lane == 0) {
      const uint32_t idesc_qk = umma_idesc(BF16, 128, kBS, false, false);
      const uint64_t qdesc0 = umma_desc_sw128(smem_u32(sQ), 16, 1024);
      const uint64_t kdesc0 = umma_desc_sw128(smem_u32(sRing), 16, 1024);
      uint32_t g = 0;
      int k = 0, ko = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++k) {
        const int pb = k & 1;
        if (!mbar_wait(&tl->plan_full[pb], (k >> 1) & 1, wait_status, 411)) break;
        const int n = tl->plan[pb].n;
        if (n > 0) {
          const int qb = ko & 1;
          if (!mbar_wait(&tl->q_full[qb], (ko >> 1) & 1, wait_status, 412)) break;
          ++ko;
          tc_fence_after();
          const uint64_t qd = qdesc0 + (uint64_t)((qb * kQBytes) >> 4);
#pragma unroll
          for (int i = 0; i < 8; ++i)   // k-step i: 16 head dims = 8 packed TMEM columns
            tc_cp_128x256b(tQ[qb] + i * 8, qd + (uint64_t)(((i >> 2) * 16384 + (i & 3) * 32) >> 4));
          tc_commit(&tl->q_stage_free[qb]);
          for (int j = 0; j < n; ++j, ++g) {
            const int st = g % kRing, sb = g % kSBuf;
            if (!mbar_wait(&tl->k_full[st], (g / kRing) & 1, wait_status, 413)) { ok = false; break; }
            // S[sb] is also P[sb]: the P V product that used it three blocks ago must be done
            if (!mbar_wait(&tl->pv_done[sb], ((g / kSBuf) & 1) ^ 1, wait_status, 414)) { ok = false; break; }
            tc_fence_after();
            const uint64_t kd = kdesc0 + (uint64_t)((st * 2 * kTile) >> 4);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              tc_mma_ts(tS0 + sb * 64, tQ[qb] + i * 8,
                        kd + (uint64_t)(((i >> 2) * 8192 + (i & 3) * 32) >> 4), idesc_qk, i ? 1u : 0u);
            tc_commit(&tl->k_free[st]);
            tc_commit(&tl->qk_done[sb]);
          }
        }
        mbar_arrive(&tl->plan_free[pb]);
      }
    }
    __syncwarp();
  } else if (warp == kWarpB) {
    // ============================================================ P V issuer
    if (lane == 0) {
      const uint32_t idesc_pv = umma_idesc(BF16, 128, kD, false, true);
      // V tile read MN-major: 16 tokens (2 KB) per k-step, the two 64-dim halves 8 KB apart
      const uint64_t vdesc0 = umma_desc_sw128(smem_u32(sRing) + kTile, 8192, 1024);
      uint32_t g = 0;
      int k = 0, ko = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++k) {
        const int pb = k & 1;
        if (!mbar_wait(&tl->plan_full[pb], (k >> 1) & 1, wait_status, 421)) break;
        const int n = tl->plan[pb].n;
        for (int j = 0; j < n; ++j, ++g) {
          const int st = g % kRing, sb = g % kSBuf;
          if (!mbar_wait(&tl->p_full[sb], (g / kSBuf) & 1, wait_status, 422)) { ok = false; break; }
          if (!mbar_wait(&tl->v_full[st], (g / kRing) & 1, wait_status, 423)) { ok = false; break; }
          // the previous tile's epilogue must have read O before it is overwritten
          if (j == 0 && !mbar_wait(&tl->o_free, (ko & 1) ^ 1, wait_status, 424)) { ok = false; break; }
          tc_fence_after();
          const uint64_t vd = vdesc0 + (uint64_t)((st * 2 * kTile) >> 4);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            tc_mma_ts(tO, tS0 + sb * 64 + packed_col(kk), vd + (uint64_t)((kk * 2048) >> 4), idesc_pv,
                      (j | kk) ? 1u : 0u);
          tc_commit(&tl->v_free[st]);
          tc_commit(&tl->pv_done[sb]);
        }
        if (n > 0) ++ko;
        if (ok) mbar_arrive(&tl->plan_free[pb]);
      }
    }
    __syncwarp();
  } else {
    // ============================================================ softmax (warps 0-7)
    const int quad = warp & 3, half = warp >> 2;
    const int r = quad * 32 + lane;       // tile row = TMEM lane
    const int t = r >> 6, rr = r & 63;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const float scale2 = p.sm_scale * kLog2e;
    uint32_t g = 0;
    uint32_t obs = 0;   // P V products whose completion this thread has observed (in order)
    // A parity wait tolerates a lag of one phase per barrier, so completions are
    // observed late (two blocks behind) instead of right before publishing P: the
    // softmax never stalls on the product it has just enabled.
    auto observe_pv = [&](uint32_t upto) -> bool {
      while (obs < upto) {
        if (!mbar_wait(&tl->pv_done[obs % kSBuf], (obs / kSBuf) & 1, wait_status, 433)) return false;
        ++obs;
      }
      return true;
    };
    int k = 0;
    bool alive = true;
    for (int item = blockIdx.x; item < n_items && alive; item += gridDim.x, ++k) {
      const int pb = k & 1;
      if (!mbar_wait(&tl->plan_full[pb], (k >> 1) & 1, wait_status, 431)) break;
      const Plan* pl = &tl->plan[pb];
      const int n = pl->n;
      const int hvalid = pl->hvalid[t], head = pl->head[t];
      const int q_row = pl->qblk[t] * kBS + rr;
      const int q_len = pl->q_len, k_len = pl->k_len, b = pl->b;
      const int qpos = pl->past + q_row;
      const bool row_ok = hvalid && q_row < q_len;
      uint8_t* orow = reinterpret_cast<uint8_t*>(p.o) +
                      ((int64_t)b * p.o_sb + (int64_t)head * p.o_sh + (int64_t)(pl->q_start + q_row) * p.o_ss) * 2 +
                      half * 128;
      float* lse_ptr = p.lse ? p.lse + (int64_t)b * p.lse_sb + (int64_t)head * p.lse_sh + pl->q_start + q_row
                             : nullptr;
      if (n == 0) {
        if (pl->valid && row_ok) {   // a tile that attends nothing: zero rows, LSE = -inf
#pragma unroll
          for (int i = 0; i < 8; ++i) reinterpret_cast<uint4*>(orow)[i] = make_uint4(0u, 0u, 0u, 0u);
          if (half == 0 && lse_ptr) *lse_ptr = -INFINITY;
        }
        mbar_arrive(&tl->plan_free[pb]);
        continue;
      }
      float m_used = -INFINITY, l = 0.f;
      for (int j = 0; j < n; ++j, ++g) {
        const int sb = g % kSBuf;
        const uint32_t tS = tS0 + sb * 64;
        if (!mbar_wait(&tl->qk_done[sb], (g / kSBuf) & 1, wait_status, 432)) { alive = false; break; }
        tc_fence_after();
        uint32_t sv[32];
        tmem_ld32(tS + lane_off + half * 32, sv);
        tmem_ld_wait();
        const uint32_t ent = pl->list[j];
        const int kbase = (int)(ent & 0x3fffu) * kBS;
        const bool att = ((ent >> (14 + t)) & 1u) != 0 && hvalid;
        // allowed columns form a prefix: kpos < k_len and (causal) kpos <= qpos
        float mx = -INFINITY;
        if (att) {
          int lim = k_len - kbase;
          if (p.causal) lim = min(lim, qpos - kbase + 1);
          lim -= half * 32;
          if (lim < 32) {
#pragma unroll
            for (int c = 0; c < 32; ++c)
              if (c >= lim) sv[c] = 0xff800000u;  // -inf
          }
          float m4[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) m4[i] = __uint_as_float(sv[i]);
#pragma unroll
          for (int c = 4; c < 32; c += 4)
#pragma unroll
            for (int i = 0; i < 4; ++i) m4[i] = fmaxf(m4[i], __uint_as_float(sv[c + i]));
          mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * scale2;
        }
        // combine with the warp that owns the other 32 columns of the same rows
        tl->xch[j & 1][half][r] = mx;
        pair_bar(quad);
        mx = fmaxf(mx, tl->xch[j & 1][half ^ 1][r]);
        float alpha = 1.f;
        bool need = false;
        if (mx != -INFINITY) {
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
        uint32_t pk[16];
        if (att && m_used != -INFINITY) {
          float sum[4] = {0.f, 0.f, 0.f, 0.f};
          const float neg_m = -m_used;
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const float p0 = ex2(fmaf(__uint_as_float(sv[2 * c]), scale2, neg_m));
            const float p1 = ex2(fmaf(__uint_as_float(sv[2 * c + 1]), scale2, neg_m));
            sum[(2 * c) & 3] += p0;
            sum[(2 * c + 1) & 3] += p1;
            pk[c] = pack2<BF16>(p0, p1);
          }
          l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
        } else {
#pragma unroll
          for (int c = 0; c < 16; ++c) pk[c] = 0u;
        }
        // packed P over the first 16 of the 32 columns this warp has just read
        tmem_st16(tS + lane_off + half * 32, pk);
        if (g >= 2 && !observe_pv(g - 1)) { alive = false; break; }
        if (any && j > 0) {
          // rescale this warp's 64 accumulator columns for the rows whose maximum moved:
          // the previous block's P V must have landed first
          if (!observe_pv(g)) { alive = false; break; }
          tc_fence_after();
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            uint32_t o[32];
            tmem_ld32(tO + lane_off + half * 64 + ch * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(tO + lane_off + half * 64 + ch * 32, o);
          }
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&tl->p_full[sb]);
      }
      if (!alive) break;
      // ---- epilogue of the tile: all its P V products must have completed
      if (!observe_pv(g)) { alive = false; break; }
      tc_fence_after();
      // total row sum = this warp's columns + the partner's
      tl->xch[n & 1][half][r] = l;
      pair_bar(quad);
      const float l_tot = l + tl->xch[n & 1][half ^ 1][r];
      const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t o[32];
        tmem_ld32(tO + lane_off + half * 64 + ch * 32, o);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            uint4 w;
            w.x = pack2<BF16>(__uint_as_float(o[c4 * 8 + 0]) * inv, __uint_as_float(o[c4 * 8 + 1]) * inv);
            w.y = pack2<BF16>(__uint_as_float(o[c4 * 8 + 2]) * inv, __uint_as_float(o[c4 * 8 + 3]) * inv);
            w.z = pack2<BF16>(__uint_as_float(o[c4 * 8 + 4]) * inv, __uint_as_float(o[c4 * 8 + 5]) * inv);
            w.w = pack2<BF16>(__uint_as_float(o[c4 * 8 + 6]) * inv, __uint_as_float(o[c4 * 8 + 7]) * inv);
            reinterpret_cast<uint4*>(orow)[ch * 4 + c4] = w;
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&tl->o_free);
      if (half == 0 && row_ok && lse_ptr) *lse_ptr = l_tot > 0.f ? (m_used + log2f(l_tot)) * kLn2 : -INFINITY;
      // the exchange slots are reused by the next tile: both partners must have read them
      pair_bar(quad);
      mbar_arrive(&tl->plan_free[pb]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kWarpA) tmem_dealloc(tmem, 512);
}

}  // namespace

bool sm100_fwd_persist_supported(const bsa_fwd_params* p) {
  // output rows are written with 16-byte stores
  return reinterpret_cast<uintptr_t>(p->o) % 16 == 0 && p->o_ss % 8 == 0 && p->o_sh % 8 == 0 &&
         p->o_sb % 8 == 0;
}

int sm100_fwd_persist(const bsa_fwd_params* p, cudaStream_t s) {
  const bool bf16 = p->dtype == BSA_BF16;
  Tmap4 tmQ, tmK, tmV;
  const uint64_t nb = p->total_q > 0 ? 1 : p->batch;
  int rc = make_tmap_4d(&tmQ, p->q, 2, kD, p->sq, p->hq, nb, p->q_ss * 2, p->q_sh * 2, p->q_sb * 2, 64, 64,
                        true, bf16);
  if (rc) return rc;
  rc = make_tmap_4d(&tmK, p->k, 2, kD, p->sk, p->hkv, nb, p->k_ss * 2, p->k_sh * 2, p->k_sb * 2, 64, 64,
                    true, bf16);
  if (rc) return rc;
  rc = make_tmap_4d(&tmV, p->v, 2, kD, p->sk, p->hkv, nb, p->v_ss * 2, p->v_sh * 2, p->v_sb * 2, 64, 64,
                    true, bf16);
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
  const int grid = n_items < sms ? n_items : sms;
  int* status = wait_status_ptr();
  if (!status) return BSA_E_CUDA;
  if (bf16) {
    auto kern = fwd_persist_kernel<true>;
    BSA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemP));
    kern<<<grid, kThreadsP, kSmemP, s>>>(tmQ, tmK, tmV, *p, mode, n_items, tiles_x, head_items, status);
  } else {
    auto kern = fwd_persist_kernel<false>;
    BSA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemP));
    kern<<<grid, kThreadsP, kSmemP, s>>>(tmQ, tmK, tmV, *p, mode, n_items, tiles_x, head_items, status);
  }
  return check_launch("fwd_persist_kernel");
}

}  // namespace bsa
