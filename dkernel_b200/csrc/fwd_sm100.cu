// Prefill / training forward on the 5th-generation tensor cores.
//
// One CTA = one 128-row query tile made of two 64-row halves that share a kv
// head, so every K/V block fetched by TMA feeds a full M=128 tcgen05.mma:
//   * PAIR_HEADS (GQA, even group size): the halves are two q heads of one kv
//     group at the same q block -- identical block lists, no wasted work;
//   * PAIR_ROWS (otherwise): the halves are two adjacent q blocks of one head;
//     the CTA walks the union of their block lists and a half that does not
//     attend a block contributes P = 0 for it.
// The per-head CSR rows of both halves are merged in shared memory (bitmaps ->
// ordered list) before the pipeline starts.
//
// Warp roles (192 threads):  warps 0-3 softmax (thread r owns tile row r = TMEM
// lane r: no cross-lane reductions at all), warp 4 TMA producer, warp 5 owns TMEM
// and issues every product from one thread.  Per kv block j:
//   S[j&1] = Q K_j^T          tcgen05.mma, A/B from 128B-swizzled smem, fp32 in TMEM
//   P = exp2(S*c - m)          softmax warps: tcgen05.ld -> registers -> bf16/fp16 ->
//                              tcgen05.st into the columns S occupied
//   O += P V_j                 tcgen05.mma, A = P from TMEM, B = V (MN-major) from smem
// The issue order is Q K_0, Q K_1, then P V_j followed at once by Q K_{j+2}: the
// tensor pipe runs one thread's products in issue order, so Q K_{j+2} may be queued
// behind P V_j without waiting for the completion that frees the columns they share.
// S is double buffered so Q K_{j+1}^T overlaps softmax j; the running maximum is
// only raised when it grows by more than 2^8 (the accumulator then gets rescaled
// in TMEM), so the correction step is rare.  Two CTAs fit per SM (about 101 KB of
// shared memory and 256 TMEM columns each), which lets one CTA's tensor-core
// work hide the other's softmax.  Math follows
// dkernel/ops/sparse_attn_fwd.py:90-165, :351-363 (base-2 online softmax, LSE).
#include <cstdlib>

#include "ptx.cuh"

namespace bsa {
namespace {

constexpr int kD = 128;
constexpr int kBS = 64;
constexpr int kFwdThreads = 192;
constexpr int kMaxList = 1024;          // kv blocks per sequence (64K tokens)
constexpr int kQBytes = 128 * kD * 2;   // 32 KB
constexpr int kKVBytes = kBS * kD * 2;  // 16 KB per K or V tile
#ifndef BSA_FWD_STAGES
#define BSA_FWD_STAGES 2
#endif
constexpr int kStagesF = BSA_FWD_STAGES;     // K and V ring depth
static_assert(kStagesF == 2, "the S/P double buffer and the K/V rings share their barriers");
constexpr float kRescaleThreshold = 8.0f;

enum { kPairHeads = 0, kPairRows = 1 };

struct FwdTail {
  uint64_t q_full;
  uint64_t k_full[kStagesF], v_full[kStagesF];
  // qk_done[j&1]: Q K_j^T has completed -> S[j&1] is readable and the K stage is free.
  // pv_done[j&1]: P V_j has completed   -> P[j&1] (= S[j&1]) and the V stage are free.
  uint64_t qk_done[2], pv_done[2], p_full[2];
  uint32_t tmem_base;
  int n_list;
  uint32_t bits[2][kMaxList / 32];
  uint32_t list[kMaxList];
};

constexpr size_t kFwdSmem = 1024 + kQBytes + kStagesF * 2 * kKVBytes + sizeof(FwdTail);

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

struct Half {
  int head, qblk, valid;
};

template <bool BF16>
__global__ void __launch_bounds__(kFwdThreads, kStagesF <= 2 ? 2 : 1)
fwd_sm100_kernel(const __grid_constant__ Tmap4 tmQ, const __grid_constant__ Tmap4 tmK,
                 const __grid_constant__ Tmap4 tmV, bsa_fwd_params p, int mode, int* wait_status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + kQBytes;  // stage s: K at s*32K, V at s*32K + 16K
  FwdTail* tl = reinterpret_cast<FwdTail*>(smem + kQBytes + kStagesF * 2 * kKVBytes);

  // A wait that gave up in an earlier launch makes every later launch return at once.  The
  // flag is loaded here and tested after the work item is known, so that its latency
  // overlaps the index arithmetic.
  const int sticky = *reinterpret_cast<volatile int*>(wait_status);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // ---------------------------------------------------------------- work item
  const int G = p.hq / p.hkv;
  const int tile_rows = mode == kPairHeads ? 64 : 128;
  int b = blockIdx.z, tile;
  if (p.total_q > 0) {
    int acc = 0, found = 0;
    tile = 0;
    for (int i = 0; i < p.batch; ++i) {
      const int len = p.q_end[i] - p.q_start[i];
      const int n = len > 0 ? (len + tile_rows - 1) / tile_rows : 0;
      if ((int)blockIdx.x < acc + n) { b = i; tile = blockIdx.x - acc; found = 1; break; }
      acc += n;
    }
    if (!found) return;
  } else {
    tile = gridDim.x - 1 - blockIdx.x;  // long rows first
  }
  const int q_start = p.q_start ? p.q_start[b] : 0;
  const int q_len = (p.q_end ? p.q_end[b] : p.sq) - q_start;
  const int k_start = p.k_start ? p.k_start[b] : 0;
  const int k_len = (p.k_end ? p.k_end[b] : p.sk) - k_start;
  if (tile * tile_rows >= q_len) return;
  const int past = (p.causal || p.row_mode == BSA_ROWS_BY_POSITION) ? k_len - q_len : 0;

  Half hf[2];
  int kvh;
  if (mode == kPairHeads) {
    const int pairs = G / 2;
    kvh = blockIdx.y / pairs;
    const int h0 = kvh * G + 2 * (blockIdx.y % pairs);
    hf[0] = {h0, tile, 1};
    hf[1] = {h0 + 1, tile, 1};
  } else {
    const int h = blockIdx.y;
    kvh = h / G;
    hf[0] = {h, 2 * tile, 1};
    hf[1] = {h, 2 * tile + 1, (2 * tile + 1) * kBS < q_len ? 1 : 0};
  }
  const int nkb = min((k_len + kBS - 1) / kBS, kMaxList);

  // CSR row bounds of both halves: the loads are issued now and consumed after the
  // barrier setup below.
  int c_beg[2] = {0, 0}, c_end[2] = {0, 0};
  const int32_t* cols_of[2] = {nullptr, nullptr};
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    if (!hf[t].valid) continue;
    const int q_first = hf[t].qblk * kBS;
    const int row = (p.row_mode == BSA_ROWS_BY_POSITION ? past + q_first : q_first) / kBS;
    if (row >= p.n_rows) continue;
    const int hp = pattern_head(hf[t].head, p.h_pat, p.hq, p.hkv);
    const int32_t* cr = p.crow + (int64_t)hp * p.crow_sh;
    cols_of[t] = p.col + (int64_t)hp * p.col_sh;
    c_beg[t] = __ldg(cr + row);
    c_end[t] = __ldg(cr + row + 1);
  }
  if (sticky != 0) return;

  // ---------------------------------------------------------------- setup
  if (warp == 0) {
    // the eleven barriers are contiguous: q_full, k_full[2], v_full[2], qk_done[2],
    // pv_done[2] (one arrival each) and p_full[2] (one arrival per softmax warp)
    if (lane < 11) {
      mbar_init(&tl->q_full + lane, lane >= 9 ? 4 : 1);
      mbar_fence_init();
    } else if (lane == 11) {
      tma_prefetch_desc(&tmQ.map);
    } else if (lane == 12) {
      tma_prefetch_desc(&tmK.map);
    } else if (lane == 13) {
      tma_prefetch_desc(&tmV.map);
    }
  } else if (tid - 32 < 2 * (kMaxList / 32)) {
    (&tl->bits[0][0])[tid - 32] = 0u;
  }
  __syncthreads();
  // The Q tile and the TMEM allocation do not depend on the block list: start them
  // now so that their latency overlaps the list construction.
  if (warp == 4 && lane == 0) {
    mbar_expect_tx(&tl->q_full, (uint32_t)(hf[0].valid + hf[1].valid) * (kQBytes / 2));
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      if (!hf[t].valid) continue;
      for (int c = 0; c < 2; ++c)
        tma_load_tile(sQ + c * 16384 + t * 8192, &tmQ, &tl->q_full, c * 64,
                      q_start + hf[t].qblk * kBS, hf[t].head, b);
    }
  }
  if (warp == 5) {
    tmem_alloc(&tl->tmem_base, 256);
    tmem_relinquish();
  }
  // union of the two halves' block lists
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int q_pos_last = past + min(hf[t].qblk * kBS + kBS, q_len) - 1;
    for (int i = c_beg[t] + tid; i < c_end[t]; i += kFwdThreads) {
      const int blk = __ldg(cols_of[t] + i);
      if (blk >= 0 && blk < nkb && !(p.causal && blk * kBS > q_pos_last))
        atomicOr(&tl->bits[t][blk >> 5], 1u << (blk & 31));
    }
  }
  __syncthreads();
  {
    // bitmaps -> ordered list.  Every warp scans the 32 word counts by itself, then the
    // warps share the words out; in a word each lane owns one bit.
    const uint32_t u0 = tl->bits[0][lane], u1 = tl->bits[1][lane];
    const uint32_t u = u0 | u1;
    const int cnt = __popc(u);
    int incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    const int base = incl - cnt;
    const uint32_t nonzero = __ballot_sync(0xffffffffu, u != 0u);
    for (int w = warp; w < 32; w += kFwdThreads / 32) {
      if (!((nonzero >> w) & 1u)) continue;
      const uint32_t uw = __shfl_sync(0xffffffffu, u, w);
      const uint32_t u0w = __shfl_sync(0xffffffffu, u0, w);
      const uint32_t u1w = __shfl_sync(0xffffffffu, u1, w);
      const int bw = __shfl_sync(0xffffffffu, base, w);
      if ((uw >> lane) & 1u)
        tl->list[bw + __popc(uw & ((1u << lane) - 1u))] =
            (uint32_t)(w * 32 + lane) | (((u0w >> lane) & 1u) << 16) | (((u1w >> lane) & 1u) << 17);
    }
    if (tid == 31) tl->n_list = incl;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const int n = tl->n_list;
  const uint32_t tmem = tl->tmem_base;
  const uint32_t tS[2] = {tmem, tmem + 64};
  const uint32_t tO = tmem + 128;

  if (n > 0 && warp == 4) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int j = 0; j < n; ++j) {
        const int s = j % kStagesF;
        const uint32_t ph = ((j / kStagesF) & 1) ^ 1;
        const int tok = k_start + (int)(tl->list[j] & 0xffffu) * kBS;
        uint8_t* kdst = sKV + s * 2 * kKVBytes;
        uint8_t* vdst = kdst + kKVBytes;
        if (!mbar_wait(&tl->qk_done[s], ph, wait_status, 201)) break;
        mbar_expect_tx(&tl->k_full[s], kKVBytes);
        tma_load_tile(kdst, &tmK, &tl->k_full[s], 0, tok, kvh, b);
        tma_load_tile(kdst + 8192, &tmK, &tl->k_full[s], 64, tok, kvh, b);
        if (!mbar_wait(&tl->pv_done[s], ph, wait_status, 202)) break;
        mbar_expect_tx(&tl->v_full[s], kKVBytes);
        tma_load_tile(vdst, &tmV, &tl->v_full[s], 0, tok, kvh, b);
        tma_load_tile(vdst + 8192, &tmV, &tl->v_full[s], 64, tok, kvh, b);
      }
    }
  } else if (n > 0 && warp == 5) {
    // ------------------------------------------------------------ MMA issuer
    // One thread issues every product, in the order  Q K_0, Q K_1, then per block j:
    // P V_j, Q K_{j+2}.  Q K_{j+2} overwrites the columns P_j sits in; it is issued right
    // behind P V_j without waiting for that product to complete, because the tensor pipe
    // executes one thread's tcgen05.mma instructions in issue order.
    // The whole warp runs this loop converged, so that descriptors and addresses stay in
    // uniform registers; only the tcgen05 instructions themselves sit under the elected lane.
    // (A single diverged lane spends about a hundred cycles of dependent scalar work per
    // product, which is more than the product takes on the tensor pipe.)
    {
      const uint32_t idesc_qk = umma_idesc(BF16, 128, kBS, false, false);
      const uint32_t idesc_pv = umma_idesc(BF16, 128, kD, false, true);
      // descriptors of the first tile of each operand; the start-address field (bits
      // 0..13, units of 16 bytes) is advanced by plain additions afterwards
      const uint64_t qdesc0 = umma_desc_sw128(smem_u32(sQ), 16, 1024);
      const uint64_t kdesc0 = umma_desc_sw128(smem_u32(sKV), 16, 1024);
      // V tile: rows = kv tokens (K of this product), 128 contiguous bytes = 64 head
      // dims (N); the two 64-dim halves are 8 KB apart (LBO); 16 tokens per k-step
      const uint64_t vdesc0 = umma_desc_sw128(smem_u32(sKV) + kKVBytes, 8192, 1024);
      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&tl->k_full[s], (j >> 1) & 1, wait_status, 204)) return false;
        tc_fence_after();
        const uint64_t db0 = kdesc0 + (uint64_t)((s * 2 * kKVBytes) >> 4);
        if (elect_one()) {
#pragma unroll
          for (int i = 0; i < 8; ++i)   // i = c * 4 + kk: sub-tile c (8 KB apart for K, 16 KB for Q), k-step kk
            tc_mma_ss(tS[s], qdesc0 + (uint64_t)(((i >> 2) * 16384 + (i & 3) * 32) >> 4),
                      db0 + (uint64_t)(((i >> 2) * 8192 + (i & 3) * 32) >> 4), idesc_qk, i ? 1u : 0u);
          tc_commit(&tl->qk_done[s]);
        }
        __syncwarp();
        return true;
      };
      bool ok = mbar_wait(&tl->q_full, 0, wait_status, 203);
      for (int j = 0; j < 2 && j < n && ok; ++j) ok = issue_qk(j);
      for (int j = 0; j < n && ok; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&tl->p_full[s], (j >> 1) & 1, wait_status, 205)) break;
        if (!mbar_wait(&tl->v_full[s], (j >> 1) & 1, wait_status, 206)) break;
        tc_fence_after();
        const uint64_t dv0 = vdesc0 + (uint64_t)((s * 2 * kKVBytes) >> 4);
        const uint32_t acc0 = j ? 1u : 0u;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            tc_mma_ts(tO, tS[s] + kk * 8, dv0 + (uint64_t)((kk * 2048) >> 4), idesc_pv, kk ? 1u : acc0);
          tc_commit(&tl->pv_done[s]);
        }
        __syncwarp();
        if (j + 2 < n) ok = issue_qk(j + 2);
      }
    }
    __syncwarp();
  } else if (n > 0) {
    // ------------------------------------------------------------ softmax (warps 0-3)
    const int r = tid;            // tile row = TMEM lane
    const int t = r >> 6;         // half
    const int rr = r & 63;
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
    const float scale2 = p.sm_scale * kLog2e;
    const Half my = t ? hf[1] : hf[0];
    const int q_row = my.qblk * kBS + rr;   // row inside the sequence
    const int qpos = past + q_row;
    float m_used = -INFINITY, l = 0.f;
    bool alive = true;
    // Completions of P V are observed in order, one phase of a barrier at a time (a parity
    // wait only means something while the waiter is at most one phase behind).  Q K_j^T was
    // issued after P V_{j-2} completed, so observing up to j-2 never blocks; P V_{j-1} is
    // only waited for when the accumulator has to be rescaled.
    int seen = 0;
    auto observe_pv = [&](int upto) {   // P V_0 .. P V_upto have completed
      while (seen <= upto) {
        if (!mbar_wait(&tl->pv_done[seen & 1], (seen >> 1) & 1, wait_status, 208)) return false;
        ++seen;
      }
      return true;
    };
    for (int j = 0; j < n; ++j) {
      if (!mbar_wait(&tl->qk_done[j & 1], (j >> 1) & 1, wait_status, 207)) { alive = false; break; }
      tc_fence_after();
      uint32_t sv[64];
      tmem_ld32(tS[j & 1] + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
      tmem_ld32(tS[j & 1] + lane_off + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
      tmem_ld_wait();
      const uint32_t ent = tl->list[j];
      const int kbase = (int)(ent & 0xffffu) * kBS;
      const bool att = ((ent >> (16 + t)) & 1u) != 0 && my.valid;
      // Allowed columns of this block form a prefix: kpos < k_len and, when causal,
      // kpos <= qpos.  Raw logits are compared (sm_scale > 0); the scale is folded
      // into the exponent's FMA.
      float mx = -INFINITY;
      if (att) {
        int lim = k_len - kbase;
        if (p.causal) lim = min(lim, qpos - kbase + 1);
        if (lim < kBS) {
#pragma unroll
          for (int c = 0; c < 64; ++c)
            if (c >= lim) sv[c] = 0xff800000u;  // -inf
        }
        float m8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) m8[i] = __uint_as_float(sv[i]);
#pragma unroll
        for (int c = 8; c < 64; c += 8)
#pragma unroll
          for (int i = 0; i < 8; ++i) m8[i] = fmaxf(m8[i], __uint_as_float(sv[c + i]));
        mx = fmaxf(fmaxf(fmaxf(m8[0], m8[1]), fmaxf(m8[2], m8[3])),
                   fmaxf(fmaxf(m8[4], m8[5]), fmaxf(m8[6], m8[7]))) * scale2;
      }
      float alpha = 1.f;
      bool need = false;
      if (att && mx != -INFINITY) {
        if (m_used == -INFINITY) {
          m_used = mx;   // first attended block of this row: O row is still exactly 0
        } else if (mx > m_used + kRescaleThreshold) {
          alpha = ex2(m_used - mx);
          m_used = mx;
          l *= alpha;
          need = true;
        }
      }
      const bool any = __any_sync(0xffffffffu, need);
      uint32_t pk[32];
      if (att && m_used != -INFINITY) {
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
        const float neg_m = -m_used;
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const float p0 = ex2(fmaf(__uint_as_float(sv[2 * c]), scale2, neg_m));
          const float p1 = ex2(fmaf(__uint_as_float(sv[2 * c + 1]), scale2, neg_m));
          sum[(2 * c) & 3] += p0;
          sum[(2 * c + 1) & 3] += p1;
          pk[c] = pack2<BF16>(p0, p1);
        }
        l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) pk[c] = 0u;
      }
      tmem_st32(tS[j & 1] + lane_off, pk);
      if (!observe_pv(any ? j - 1 : j - 2)) { alive = false; break; }
      if (any && j > 0) {
        // rescale the accumulator rows whose maximum moved (P V_{j-1} has landed)
        tc_fence_after();
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t o[32];
          tmem_ld32(tO + lane_off + ch * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(tO + lane_off + ch * 32, o);
        }
      }
      // tcgen05.wait::st is warp-wide: after it every lane's P row is in TMEM, so one
      // arrival per warp publishes them
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tl->p_full[j & 1]);
    }
    // ---- epilogue: O / l -> registers -> swizzled smem (the Q tile is dead) -> global
    if (alive) alive = observe_pv(n - 1);
    tc_fence_after();
    if (alive) {
      // ---- epilogue: each thread normalises its own row and stores it straight from
      // registers, 64 contiguous bytes per 32-column chunk
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool row_ok = my.valid && q_row < q_len;
      uint8_t* orow = reinterpret_cast<uint8_t*>(p.o) +
                      ((int64_t)b * p.o_sb + (int64_t)my.head * p.o_sh + (int64_t)(q_start + q_row) * p.o_ss) * 2;
      const bool wide = reinterpret_cast<uintptr_t>(p.o) % 16 == 0 && p.o_ss % 8 == 0 &&
                        p.o_sh % 8 == 0 && p.o_sb % 8 == 0;   // rows start on 16-byte boundaries
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t o[32];
        tmem_ld32(tO + lane_off + ch * 32, o);
        tmem_ld_wait();
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
          w[i] = pack2<BF16>(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
        if (row_ok) {
          if (wide) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              *reinterpret_cast<uint4*>(orow + ch * 64 + i * 16) =
                  make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              *reinterpret_cast<uint2*>(orow + ch * 64 + i * 8) = make_uint2(w[2 * i], w[2 * i + 1]);
          }
        }
      }
      if (p.lse && row_ok)
        p.lse[(int64_t)b * p.lse_sb + (int64_t)my.head * p.lse_sh + q_start + q_row] =
            l > 0.f ? (m_used + log2f(l)) * kLn2 : -INFINITY;
    }
  } else if (warp == 4) {
    // nothing to attend: the Q tile is still in flight and must land before the CTA exits
    if (lane == 0) mbar_wait(&tl->q_full, 0, wait_status, 211);
  } else if (warp < 4) {
    // no attended block at all: zero rows, LSE = -inf
    const int r = tid, t = r >> 6;
    const Half my = t ? hf[1] : hf[0];
    const int q_row = my.qblk * kBS + (r & 63);
    if (my.valid && q_row < q_len) {
      uint4* dst = reinterpret_cast<uint4*>(
          reinterpret_cast<uint8_t*>(p.o) +
          ((int64_t)b * p.o_sb + (int64_t)my.head * p.o_sh + (int64_t)(q_start + q_row) * p.o_ss) * 2);
      // rows are only guaranteed 8-byte aligned
      uint2* d2 = reinterpret_cast<uint2*>(dst);
      for (int i = 0; i < 32; ++i) d2[i] = make_uint2(0u, 0u);
      if (p.lse)
        p.lse[(int64_t)b * p.lse_sb + (int64_t)my.head * p.lse_sh + q_start + q_row] = -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem, 256);
}

}  // namespace

bool sm100_fwd_supported(const bsa_fwd_params* p, const char** why) {
  auto no = [&](const char* w) { *why = w; return false; };
  if (!(p->dtype == BSA_F16 || p->dtype == BSA_BF16)) return no("dtype is not f16/bf16");
  if (p->d != kD) return no("head dim is not 128");
  if (p->block_size != kBS) return no("block size is not 64");
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

int sm100_fwd(const bsa_fwd_params* p, cudaStream_t s) {
  // The persistent kernel (two CTAs per SM walking the tile list) serves every call;
  // BSA_FWD_TILED=1 selects the one-tile-per-CTA kernel below for comparison runs.
  static const bool tiled = getenv("BSA_FWD_TILED") != nullptr;
  if (!tiled && sm100_fwd_persist_supported(p)) return sm100_fwd_persist(p, s);
  const bool bf16 = p->dtype == BSA_BF16;
  Tmap4 tmQ, tmK, tmV;
  int rc = make_tmap_4d(&tmQ, p->q, 2, kD, p->sq, p->hq, p->total_q > 0 ? 1 : p->batch, p->q_ss * 2,
                        p->q_sh * 2, p->q_sb * 2, 64, 64, true, bf16);
  if (rc) return rc;
  rc = make_tmap_4d(&tmK, p->k, 2, kD, p->sk, p->hkv, p->total_q > 0 ? 1 : p->batch, p->k_ss * 2,
                    p->k_sh * 2, p->k_sb * 2, 64, 64, true, bf16);
  if (rc) return rc;
  rc = make_tmap_4d(&tmV, p->v, 2, kD, p->sk, p->hkv, p->total_q > 0 ? 1 : p->batch, p->v_ss * 2,
                    p->v_sh * 2, p->v_sb * 2, 64, 64, true, bf16);
  if (rc) return rc;
  const int G = p->hq / p->hkv;
  // Two heads share a tile only when they share a block list (one pattern for all heads
  // or one per kv head): with per-head patterns the union of two heads' lists would spend
  // half of the tensor work of every unshared block on an unattended half.  Two adjacent
  // row blocks of one head share all but the two ends of their lists.
  const int mode = (G % 2 == 0 && p->h_pat != p->hq) ? kPairHeads : kPairRows;
  const int tile_rows = mode == kPairHeads ? 64 : 128;
  const int head_items = mode == kPairHeads ? p->hq / 2 : p->hq;
  dim3 grid;
  if (p->total_q > 0)
    grid = dim3(cdiv_i(p->total_q, tile_rows) + p->batch, head_items, 1);
  else
    grid = dim3(cdiv_i(p->sq, tile_rows), head_items, p->batch);
  int* status = wait_status_ptr();
  if (!status) return BSA_E_CUDA;
  if (bf16) {
    auto kern = fwd_sm100_kernel<true>;
    BSA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFwdSmem));
    kern<<<grid, kFwdThreads, kFwdSmem, s>>>(tmQ, tmK, tmV, *p, mode, status);
  } else {
    auto kern = fwd_sm100_kernel<false>;
    BSA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFwdSmem));
    kern<<<grid, kFwdThreads, kFwdSmem, s>>>(tmQ, tmK, tmV, *p, mode, status);
  }
  return check_launch("fwd_sm100_kernel");
}

}  // namespace bsa
