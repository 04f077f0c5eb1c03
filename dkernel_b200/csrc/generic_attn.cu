// Generic block-sparse attention kernels (forward, backward) on CUDA cores with
// fp32 accumulation.  They serve every shape the tensor-core kernels do not
// (fp32 inputs, head dims other than 128, block sizes other than 64, ...) and
// act as the on-device cross-check of the tcgen05 kernels.  Same math as
// dkernel/ops/sparse_attn_fwd.py:90-165 and dkernel/ops/sparse_attn_bwd.py:86-170,
// :329-419, with -inf masking and guarded maxima so that empty rows give O=0,
// LSE=-inf instead of NaN.
//
// Tiling: a CTA of 256 threads owns TILE query rows (forward, dQ) or TILE key
// rows (dK/dV); TILE = min(block_size, 64), 32 at most when D > 128.  Operand
// tiles live in shared memory as fp32 with a row stride of DP+4 floats
// (DP = D rounded up to 8), which makes the float4 reads of 8 consecutive rows
// conflict-free.  Thread t = (rg, cg) = (t / 16, t % 16) owns rows rg + 16*i and
// columns cg + 16*j of every product.
#include "common.cuh"

namespace bsa {
namespace {

constexpr int kThreads = 256;

struct SeqInfo {
  int q_start, q_len, k_start, k_len, past;
};

__device__ __forceinline__ SeqInfo seq_info(const bsa_fwd_params& p, int b) {
  SeqInfo s;
  s.q_start = p.q_start ? p.q_start[b] : 0;
  s.q_len = (p.q_end ? p.q_end[b] : p.sq) - s.q_start;
  s.k_start = p.k_start ? p.k_start[b] : 0;
  s.k_len = (p.k_end ? p.k_end[b] : p.sk) - s.k_start;
  s.past = (p.causal || p.row_mode == BSA_ROWS_BY_POSITION) ? s.k_len - s.q_len : 0;
  return s;
}

// Packed batches: tile number `flat` over all sequences -> (sequence, tile).
__device__ __forceinline__ bool flat_tile_to_seq(const bsa_fwd_params& p, int tile, int flat, int* b,
                                                 int* qt) {
  int acc = 0;
  for (int i = 0; i < p.batch; ++i) {
    const int len = (p.q_end ? p.q_end[i] : p.sq) - (p.q_start ? p.q_start[i] : 0);
    const int n = len > 0 ? (len + tile - 1) / tile : 0;
    if (flat < acc + n) {
      *b = i;
      *qt = flat - acc;
      return true;
    }
    acc += n;
  }
  return false;
}

// rows [row0, row0+TILE) of a (rows x D) matrix with row stride `rs` -> smem
// fp32 [TILE][LD]; rows >= n_valid and columns >= D are zero.
template <typename T, int TILE>
__device__ __forceinline__ void load_tile(float* dst, int LD, const T* src, int64_t rs, int row0,
                                          int n_valid, int D, int DP) {
  for (int idx = threadIdx.x; idx < TILE * DP; idx += kThreads) {
    const int r = idx / DP, d = idx - r * DP;
    const int row = row0 + r;
    float v = 0.f;
    if (row >= 0 && row < n_valid && d < D) v = Elem<T>::to_f(src[(int64_t)row * rs + d]);
    dst[r * LD + d] = v;
  }
}

// c[i][j] = sum_d A[rg+16i][d] * B[cg+16j][d]
template <int RM>
__device__ __forceinline__ void gemm_nt(const float* A, const float* B, int LD, int DP,
                                        float (&c)[RM][RM]) {
  const int rg = threadIdx.x >> 4, cg = threadIdx.x & 15;
#pragma unroll
  for (int i = 0; i < RM; ++i)
#pragma unroll
    for (int j = 0; j < RM; ++j) c[i][j] = 0.f;
  for (int d = 0; d < DP; d += 4) {
    float4 a[RM], b[RM];
#pragma unroll
    for (int i = 0; i < RM; ++i) a[i] = *reinterpret_cast<const float4*>(A + (rg + 16 * i) * LD + d);
#pragma unroll
    for (int j = 0; j < RM; ++j) b[j] = *reinterpret_cast<const float4*>(B + (cg + 16 * j) * LD + d);
#pragma unroll
    for (int i = 0; i < RM; ++i)
#pragma unroll
      for (int j = 0; j < RM; ++j)
        c[i][j] += a[i].x * b[j].x + a[i].y * b[j].y + a[i].z * b[j].z + a[i].w * b[j].w;
  }
}

// acc[i][t] += sum_j P(rg+16i, j) * B[j][cg+16t];  P is TILE x TILE with row
// stride TILE+1, read transposed when TRANS.
template <int TILE, int RM, bool TRANS>
__device__ __forceinline__ void gemm_acc(const float* P, const float* B, int LD, int DP,
                                         float (&acc)[RM][16]) {
  const int rg = threadIdx.x >> 4, cg = threadIdx.x & 15;
  for (int j = 0; j < TILE; ++j) {
    float pv[RM];
#pragma unroll
    for (int i = 0; i < RM; ++i)
      pv[i] = TRANS ? P[j * (TILE + 1) + rg + 16 * i] : P[(rg + 16 * i) * (TILE + 1) + j];
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      if (cg + 16 * t < DP) {
        const float b = B[j * LD + cg + 16 * t];
#pragma unroll
        for (int i = 0; i < RM; ++i) acc[i][t] += pv[i] * b;
      }
    }
  }
}

// ------------------------------------------------------------------ forward
template <typename T, int TILE>
__global__ void __launch_bounds__(kThreads) generic_fwd_kernel(bsa_fwd_params p, int DP) {
  constexpr int RM = TILE / 16;
  constexpr int TPR = kThreads / TILE;  // threads per row in the softmax phase
  extern __shared__ __align__(16) float smem[];
  const int LD = DP + 4;
  float* Qs = smem;
  float* KVs = Qs + TILE * LD;
  float* Ss = KVs + TILE * LD;
  float* m_s = Ss + TILE * (TILE + 1);
  float* l_s = m_s + TILE;
  float* a_s = l_s + TILE;

  int qt = blockIdx.x, b = blockIdx.z;
  const int h = blockIdx.y;
  if (p.total_q > 0 && !flat_tile_to_seq(p, TILE, blockIdx.x, &b, &qt)) return;
  const SeqInfo si = seq_info(p, b);
  const int q0 = qt * TILE;
  if (q0 >= si.q_len) return;
  const int hk = h / (p.hq / p.hkv);
  const int hp = pattern_head(h, p.h_pat, p.hq, p.hkv);
  const int bs = p.block_size;
  const int row = (p.row_mode == BSA_ROWS_BY_POSITION ? (si.past + q0) : q0) / bs;
  const int tid = threadIdx.x, rg = tid >> 4, cg = tid & 15;

  const T* qb = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_sb + (int64_t)h * p.q_sh +
                (int64_t)si.q_start * p.q_ss;
  const T* kb = reinterpret_cast<const T*>(p.k) + (int64_t)b * p.k_sb + (int64_t)hk * p.k_sh +
                (int64_t)si.k_start * p.k_ss;
  const T* vb = reinterpret_cast<const T*>(p.v) + (int64_t)b * p.v_sb + (int64_t)hk * p.v_sh +
                (int64_t)si.k_start * p.v_ss;

  load_tile<T, TILE>(Qs, LD, qb, p.q_ss, q0, si.q_len, p.d, DP);
  for (int i = tid; i < TILE; i += kThreads) { m_s[i] = -INFINITY; l_s[i] = 0.f; }
  float acc[RM][16];
#pragma unroll
  for (int i = 0; i < RM; ++i)
#pragma unroll
    for (int t = 0; t < 16; ++t) acc[i][t] = 0.f;

  int c_beg = 0, c_end = 0;
  if (row < p.n_rows) {
    const int32_t* cr = p.crow + (int64_t)hp * p.crow_sh;
    c_beg = cr[row];
    c_end = cr[row + 1];
  }
  const int32_t* cols = p.col + (int64_t)hp * p.col_sh;
  const float scale2 = p.sm_scale * kLog2e;
  const int q_pos_last = si.past + min(q0 + TILE, si.q_len) - 1;
  const int subs = bs / TILE;

  for (int ci = c_beg; ci < c_end; ++ci) {
    const int cblk = cols[ci];
    for (int sub = 0; sub < subs; ++sub) {
      const int k0 = cblk * bs + sub * TILE;
      if (k0 >= si.k_len) break;
      if (p.causal && k0 > q_pos_last) break;
      __syncthreads();  // previous tile's readers of KVs / Ss are done
      load_tile<T, TILE>(KVs, LD, kb, p.k_ss, k0, si.k_len, p.d, DP);
      __syncthreads();
      float c[RM][RM];
      gemm_nt<RM>(Qs, KVs, LD, DP, c);
#pragma unroll
      for (int i = 0; i < RM; ++i)
#pragma unroll
        for (int j = 0; j < RM; ++j) {
          const int r = rg + 16 * i, cc = cg + 16 * j;
          const int qpos = si.past + q0 + r, kpos = k0 + cc;
          const bool ok = kpos < si.k_len && (!p.causal || kpos <= qpos);
          Ss[r * (TILE + 1) + cc] = ok ? c[i][j] * scale2 : -INFINITY;
        }
      __syncthreads();
      // V can stream in while the softmax runs on Ss
      load_tile<T, TILE>(KVs, LD, vb, p.v_ss, k0, si.k_len, p.d, DP);
      {
        const int r = tid / TPR, sub_t = tid % TPR;
        float mx = -INFINITY;
        for (int j = sub_t; j < TILE; j += TPR) mx = fmaxf(mx, Ss[r * (TILE + 1) + j]);
#pragma unroll
        for (int o = TPR / 2; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float m_old = m_s[r];
        const float m_new = fmaxf(m_old, mx);
        const float m_safe = m_new == -INFINITY ? 0.f : m_new;
        float sum = 0.f;
        for (int j = sub_t; j < TILE; j += TPR) {
          const float pv = exp2f(Ss[r * (TILE + 1) + j] - m_safe);
          Ss[r * (TILE + 1) + j] = pv;
          sum += pv;
        }
#pragma unroll
        for (int o = TPR / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (sub_t == 0) {
          const float alpha = exp2f(m_old - m_safe);  // m_old = -inf -> 0
          a_s[r] = alpha;
          l_s[r] = l_s[r] * alpha + sum;
          m_s[r] = m_new;
        }
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < RM; ++i) {
        const float alpha = a_s[rg + 16 * i];
#pragma unroll
        for (int t = 0; t < 16; ++t) acc[i][t] *= alpha;
      }
      gemm_acc<TILE, RM, false>(Ss, KVs, LD, DP, acc);
    }
  }
  __syncthreads();
  T* ob = reinterpret_cast<T*>(p.o) + (int64_t)b * p.o_sb + (int64_t)h * p.o_sh +
          (int64_t)si.q_start * p.o_ss;
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    const int r = rg + 16 * i;
    if (q0 + r < si.q_len) {
      const float l = l_s[r];
      const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        const int d = cg + 16 * t;
        if (d < p.d) ob[(int64_t)(q0 + r) * p.o_ss + d] = Elem<T>::from_f(acc[i][t] * inv);
      }
    }
  }
  if (p.lse) {
    for (int r = tid; r < TILE; r += kThreads) {
      if (q0 + r < si.q_len) {
        const float l = l_s[r];
        p.lse[(int64_t)b * p.lse_sb + (int64_t)h * p.lse_sh + si.q_start + q0 + r] =
            l > 0.f ? (m_s[r] + log2f(l)) * kLn2 : -INFINITY;
      }
    }
  }
}

// ------------------------------------------------------------------ backward
// delta[b,h,i] = sum_d O*dO - dLSE   (dkernel/ops/sparse_attn_bwd.py:73-80)
template <typename T>
__global__ void bwd_delta_kernel(bsa_bwd_params bp) {
  const bsa_fwd_params& p = bp.f;
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long total = (long long)p.batch * p.hq * p.sq;
  if (w >= total) return;
  const int i = (int)(w % p.sq);
  const int h = (int)((w / p.sq) % p.hq);
  const int b = (int)(w / ((long long)p.sq * p.hq));
  const T* o = reinterpret_cast<const T*>(p.o) + (int64_t)b * p.o_sb + (int64_t)h * p.o_sh +
               (int64_t)i * p.o_ss;
  const T* g = reinterpret_cast<const T*>(bp.d_o) + (int64_t)b * bp.do_sb + (int64_t)h * bp.do_sh +
               (int64_t)i * bp.do_ss;
  float s = 0.f;
  for (int d = lane; d < p.d; d += 32) s += Elem<T>::to_f(o[d]) * Elem<T>::to_f(g[d]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) {
    if (bp.d_lse) s -= bp.d_lse[(int64_t)b * p.lse_sb + (int64_t)h * p.lse_sh + i];
    bp.delta[w] = s;
  }
}

// P and dS of one (q tile, k tile) pair into shared memory.
//   P  = exp(S*scale - LSE),  dS = P * (dO.V^T - delta) * scale
template <int TILE, int RM>
__device__ __forceinline__ void tile_p_ds(const float* Qs, const float* dOs, const float* Ks,
                                          const float* Vs, int LD, int DP, float* Ps, float* dSs,
                                          const float* lse_s, const float* delta_s, float sm_scale,
                                          int q_pos0, int k0, int q_valid, int k_len, bool causal) {
  const int rg = threadIdx.x >> 4, cg = threadIdx.x & 15;
  float s[RM][RM], dp[RM][RM];
  gemm_nt<RM>(Qs, Ks, LD, DP, s);
  gemm_nt<RM>(dOs, Vs, LD, DP, dp);
#pragma unroll
  for (int i = 0; i < RM; ++i)
#pragma unroll
    for (int j = 0; j < RM; ++j) {
      const int r = rg + 16 * i, cc = cg + 16 * j;
      const int kpos = k0 + cc;
      const bool ok = r < q_valid && kpos < k_len && (!causal || kpos <= q_pos0 + r);
      const float lse = lse_s[r];
      float pv = 0.f;
      if (ok && lse != -INFINITY) pv = exp2f(s[i][j] * sm_scale * kLog2e - lse * kLog2e);
      Ps[r * (TILE + 1) + cc] = pv;
      dSs[r * (TILE + 1) + cc] = pv * (dp[i][j] - delta_s[r]) * sm_scale;
    }
}

template <typename T, int TILE>
__global__ void __launch_bounds__(kThreads) generic_bwd_dq_kernel(bsa_bwd_params bp, int DP) {
  constexpr int RM = TILE / 16;
  const bsa_fwd_params& p = bp.f;
  extern __shared__ __align__(16) float smem[];
  const int LD = DP + 4;
  float* Qs = smem;
  float* dOs = Qs + TILE * LD;
  float* Ks = dOs + TILE * LD;
  float* Vs = Ks + TILE * LD;
  float* Ps = Vs + TILE * LD;
  float* dSs = Ps + TILE * (TILE + 1);
  float* lse_s = dSs + TILE * (TILE + 1);
  float* delta_s = lse_s + TILE;

  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = qt * TILE;
  if (q0 >= p.sq) return;
  const int hk = h / (p.hq / p.hkv);
  const int hp = pattern_head(h, p.h_pat, p.hq, p.hkv);
  const int bs = p.block_size;
  const int past = p.causal ? p.sk - p.sq : 0;
  const int row = q0 / bs;
  const int tid = threadIdx.x, rg = tid >> 4, cg = tid & 15;
  const int q_valid = min(TILE, p.sq - q0);

  const T* qb = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_sb + (int64_t)h * p.q_sh;
  const T* gb = reinterpret_cast<const T*>(bp.d_o) + (int64_t)b * bp.do_sb + (int64_t)h * bp.do_sh;
  const T* kb = reinterpret_cast<const T*>(p.k) + (int64_t)b * p.k_sb + (int64_t)hk * p.k_sh;
  const T* vb = reinterpret_cast<const T*>(p.v) + (int64_t)b * p.v_sb + (int64_t)hk * p.v_sh;
  load_tile<T, TILE>(Qs, LD, qb, p.q_ss, q0, p.sq, p.d, DP);
  load_tile<T, TILE>(dOs, LD, gb, bp.do_ss, q0, p.sq, p.d, DP);
  for (int i = tid; i < TILE; i += kThreads) {
    const bool ok = q0 + i < p.sq;
    lse_s[i] = ok ? p.lse[(int64_t)b * p.lse_sb + (int64_t)h * p.lse_sh + q0 + i] : -INFINITY;
    delta_s[i] = ok ? bp.delta[((int64_t)b * p.hq + h) * p.sq + q0 + i] : 0.f;
  }
  float acc[RM][16];
#pragma unroll
  for (int i = 0; i < RM; ++i)
#pragma unroll
    for (int t = 0; t < 16; ++t) acc[i][t] = 0.f;

  int c_beg = 0, c_end = 0;
  if (row < p.n_rows) {
    const int32_t* cr = p.crow + (int64_t)hp * p.crow_sh;
    c_beg = cr[row];
    c_end = cr[row + 1];
  }
  const int32_t* cols = p.col + (int64_t)hp * p.col_sh;
  const int q_pos_last = past + q0 + q_valid - 1;
  const int subs = bs / TILE;
  for (int ci = c_beg; ci < c_end; ++ci) {
    const int cblk = cols[ci];
    for (int sub = 0; sub < subs; ++sub) {
      const int k0 = cblk * bs + sub * TILE;
      if (k0 >= p.sk) break;
      if (p.causal && k0 > q_pos_last) break;
      __syncthreads();
      load_tile<T, TILE>(Ks, LD, kb, p.k_ss, k0, p.sk, p.d, DP);
      load_tile<T, TILE>(Vs, LD, vb, p.v_ss, k0, p.sk, p.d, DP);
      __syncthreads();
      tile_p_ds<TILE, RM>(Qs, dOs, Ks, Vs, LD, DP, Ps, dSs, lse_s, delta_s, p.sm_scale, past + q0,
                          k0, q_valid, p.sk, p.causal != 0);
      __syncthreads();
      gemm_acc<TILE, RM, false>(dSs, Ks, LD, DP, acc);
    }
  }
  T* dqb = reinterpret_cast<T*>(bp.dq) + (int64_t)b * bp.dq_sb + (int64_t)h * bp.dq_sh;
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    const int r = rg + 16 * i;
    if (r < q_valid) {
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        const int d = cg + 16 * t;
        if (d < p.d) dqb[(int64_t)(q0 + r) * bp.dq_ss + d] = Elem<T>::from_f(acc[i][t]);
      }
    }
  }
}

// One CTA per (k tile, kv head, batch): K, V resident, the q heads of the group
// and their CSC row lists are walked in turn, so dK/dV are written exactly once.
template <typename T, int TILE>
__global__ void __launch_bounds__(kThreads) generic_bwd_dkdv_kernel(bsa_bwd_params bp, int DP) {
  constexpr int RM = TILE / 16;
  const bsa_fwd_params& p = bp.f;
  extern __shared__ __align__(16) float smem[];
  const int LD = DP + 4;
  float* Qs = smem;
  float* dOs = Qs + TILE * LD;
  float* Ks = dOs + TILE * LD;
  float* Vs = Ks + TILE * LD;
  float* Ps = Vs + TILE * LD;
  float* dSs = Ps + TILE * (TILE + 1);
  float* lse_s = dSs + TILE * (TILE + 1);
  float* delta_s = lse_s + TILE;

  const int kt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int k0 = kt * TILE;
  if (k0 >= p.sk) return;
  const int bs = p.block_size;
  const int past = p.causal ? p.sk - p.sq : 0;
  const int colblk = k0 / bs;
  const int tid = threadIdx.x, rg = tid >> 4, cg = tid & 15;
  const int k_valid = min(TILE, p.sk - k0);
  const int group = p.hq / p.hkv;

  const T* kb = reinterpret_cast<const T*>(p.k) + (int64_t)b * p.k_sb + (int64_t)hk * p.k_sh;
  const T* vb = reinterpret_cast<const T*>(p.v) + (int64_t)b * p.v_sb + (int64_t)hk * p.v_sh;
  load_tile<T, TILE>(Ks, LD, kb, p.k_ss, k0, p.sk, p.d, DP);
  load_tile<T, TILE>(Vs, LD, vb, p.v_ss, k0, p.sk, p.d, DP);
  float dk[RM][16], dv[RM][16];
#pragma unroll
  for (int i = 0; i < RM; ++i)
#pragma unroll
    for (int t = 0; t < 16; ++t) { dk[i][t] = 0.f; dv[i][t] = 0.f; }
  const int subs = bs / TILE;

  for (int g = 0; g < group; ++g) {
    const int h = hk * group + g;
    const int hp = pattern_head(h, p.h_pat, p.hq, p.hkv);
    int r_beg = 0, r_end = 0;
    if (colblk < bp.n_cols) {
      const int32_t* cc = bp.ccol + (int64_t)hp * bp.ccol_sh;
      r_beg = cc[colblk];
      r_end = cc[colblk + 1];
    }
    const int32_t* rows = bp.row + (int64_t)hp * bp.row_sh;
    const T* qb = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_sb + (int64_t)h * p.q_sh;
    const T* gb = reinterpret_cast<const T*>(bp.d_o) + (int64_t)b * bp.do_sb + (int64_t)h * bp.do_sh;
    for (int ri = r_beg; ri < r_end; ++ri) {
      const int rblk = rows[ri];
      for (int sub = 0; sub < subs; ++sub) {
        const int q0 = rblk * bs + sub * TILE;
        if (q0 >= p.sq) break;
        const int q_valid = min(TILE, p.sq - q0);
        if (p.causal && k0 > past + q0 + q_valid - 1) continue;
        __syncthreads();
        load_tile<T, TILE>(Qs, LD, qb, p.q_ss, q0, p.sq, p.d, DP);
        load_tile<T, TILE>(dOs, LD, gb, bp.do_ss, q0, p.sq, p.d, DP);
        for (int i = tid; i < TILE; i += kThreads) {
          const bool ok = q0 + i < p.sq;
          lse_s[i] = ok ? p.lse[(int64_t)b * p.lse_sb + (int64_t)h * p.lse_sh + q0 + i] : -INFINITY;
          delta_s[i] = ok ? bp.delta[((int64_t)b * p.hq + h) * p.sq + q0 + i] : 0.f;
        }
        __syncthreads();
        tile_p_ds<TILE, RM>(Qs, dOs, Ks, Vs, LD, DP, Ps, dSs, lse_s, delta_s, p.sm_scale,
                            past + q0, k0, q_valid, p.sk, p.causal != 0);
        __syncthreads();
        gemm_acc<TILE, RM, true>(Ps, dOs, LD, DP, dv);
        gemm_acc<TILE, RM, true>(dSs, Qs, LD, DP, dk);
      }
    }
  }
  T* dkb = reinterpret_cast<T*>(bp.dk) + (int64_t)b * bp.dk_sb + (int64_t)hk * bp.dk_sh;
  T* dvb = reinterpret_cast<T*>(bp.dv) + (int64_t)b * bp.dv_sb + (int64_t)hk * bp.dv_sh;
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    const int r = rg + 16 * i;
    if (r < k_valid) {
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        const int d = cg + 16 * t;
        if (d < p.d) {
          dkb[(int64_t)(k0 + r) * bp.dk_ss + d] = Elem<T>::from_f(dk[i][t]);
          dvb[(int64_t)(k0 + r) * bp.dv_ss + d] = Elem<T>::from_f(dv[i][t]);
        }
      }
    }
  }
}

int pick_tile(int block_size, int d) {
  int t = block_size < 64 ? block_size : 64;
  if (d > 128 && t > 32) t = 32;
  return t;
}

template <typename T, int TILE>
int launch_fwd(const bsa_fwd_params* p, cudaStream_t s) {
  const int DP = (p->d + 7) / 8 * 8;
  const size_t smem = sizeof(float) * (2 * TILE * (DP + 4) + TILE * (TILE + 1) + 3 * TILE);
  auto kern = generic_fwd_kernel<T, TILE>;
  BSA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(cdiv_i(p->sq, TILE), p->hq, p->batch);
  if (p->total_q > 0) grid = dim3(cdiv_i(p->total_q, TILE) + p->batch, p->hq, 1);
  kern<<<grid, kThreads, smem, s>>>(*p, DP);
  return check_launch("generic_fwd_kernel");
}

template <typename T, int TILE>
int launch_bwd(const bsa_bwd_params* bp, cudaStream_t s) {
  const bsa_fwd_params* p = &bp->f;
  const int DP = (p->d + 7) / 8 * 8;
  const size_t smem = sizeof(float) * (4 * TILE * (DP + 4) + 2 * TILE * (TILE + 1) + 2 * TILE);
  {
    const long long rows = (long long)p->batch * p->hq * p->sq;
    bwd_delta_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(*bp);
    int rc = check_launch("bwd_delta_kernel");
    if (rc) return rc;
  }
  auto kq = generic_bwd_dq_kernel<T, TILE>;
  BSA_CHECK_CUDA(cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kq<<<dim3(cdiv_i(p->sq, TILE), p->hq, p->batch), kThreads, smem, s>>>(*bp, DP);
  int rc = check_launch("generic_bwd_dq_kernel");
  if (rc) return rc;
  auto kk = generic_bwd_dkdv_kernel<T, TILE>;
  BSA_CHECK_CUDA(cudaFuncSetAttribute(kk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kk<<<dim3(cdiv_i(p->sk, TILE), p->hkv, p->batch), kThreads, smem, s>>>(*bp, DP);
  return check_launch("generic_bwd_dkdv_kernel");
}

template <typename T>
int dispatch_fwd(const bsa_fwd_params* p, cudaStream_t s) {
  switch (pick_tile(p->block_size, p->d)) {
    case 16: return launch_fwd<T, 16>(p, s);
    case 32: return launch_fwd<T, 32>(p, s);
    default: return launch_fwd<T, 64>(p, s);
  }
}
template <typename T>
int dispatch_bwd(const bsa_bwd_params* p, cudaStream_t s) {
  switch (pick_tile(p->f.block_size, p->f.d)) {
    case 16: return launch_bwd<T, 16>(p, s);
    case 32: return launch_bwd<T, 32>(p, s);
    default: return launch_bwd<T, 64>(p, s);
  }
}

}  // namespace

int generic_fwd(const bsa_fwd_params* p, cudaStream_t s) {
  if (p->d > 256) {
    set_error("bsa_fwd: head dim %d > 256 is not supported", p->d);
    return BSA_E_UNSUPPORTED;
  }
  if (p->batch == 0 || p->sq == 0 || p->hq == 0) return BSA_OK;
  switch (p->dtype) {
    case BSA_F16: return dispatch_fwd<__half>(p, s);
    case BSA_BF16: return dispatch_fwd<__nv_bfloat16>(p, s);
    case BSA_F32: return dispatch_fwd<float>(p, s);
  }
  set_error("bsa_fwd: unknown dtype %d", p->dtype);
  return BSA_E_BADARG;
}

int generic_bwd(const bsa_bwd_params* p, cudaStream_t s) {
  if (p->f.d > 256) {
    set_error("bsa_bwd: head dim %d > 256 is not supported", p->f.d);
    return BSA_E_UNSUPPORTED;
  }
  if (p->f.batch == 0 || p->f.sq == 0 || p->f.hq == 0) return BSA_OK;
  switch (p->f.dtype) {
    case BSA_F16: return dispatch_bwd<__half>(p, s);
    case BSA_BF16: return dispatch_bwd<__nv_bfloat16>(p, s);
    case BSA_F32: return dispatch_bwd<float>(p, s);
  }
  set_error("bsa_bwd: unknown dtype %d", p->f.dtype);
  return BSA_E_BADARG;
}

}  // namespace bsa
