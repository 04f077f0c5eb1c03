// Device-side sparse-layout builder: local-stride block mask, CSR/CSC row
// pointers and -1 padded index lists.  Integer work, one pass over the mask per
// kernel; bit-exact with dkernel/utils.py:19-65 and :143-220 of the reference.
#include "common.cuh"

namespace bsa {

namespace {

__device__ __forceinline__ int pymod(int a, int b) {
  int r = a % b;
  return r < 0 ? r + b : r;
}

// One thread per mask element (h, m, n); n fastest so stores coalesce.
__global__ void local_stride_mask_kernel(bsa_local_stride_params p, uint8_t* __restrict__ mask) {
  const int rows = p.q_blocks - p.trim_q_blocks;
  const long long total = (long long)p.num_heads * rows * p.kv_blocks;
  const int q_per_kv = p.num_heads / p.num_kv_heads;
  const int sparse_heads = p.num_kv_heads - p.num_dense_heads;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int n = (int)(i % p.kv_blocks);
    const long long t = i / p.kv_blocks;
    const int m = (int)(t % rows) + p.trim_q_blocks;
    const int h = (int)(t / rows);
    const int kvh = h / q_per_kv;
    const int qp = p.q_start_block + m;
    const int kp = p.kv_start_block + n;
    bool on;
    if (p.absolute_vert) {
      // dkernel/utils.py:187-194
      const bool vert = kvh < sparse_heads
                            ? pymod(p.kv_start_block + n + kvh * p.head_sliding_step +
                                        p.head_sliding_offset, p.vert_stride) == 0
                            : true;
      const bool local = (qp - kp) < p.local_left && (kp - qp) < p.local_right;
      on = vert || local;
    } else {
      // dkernel/utils.py:196-210
      int left = (qp - kp) - p.local_left + 1;
      left = left > 0 ? left : 0;
      int right = (kp - qp) - p.local_right + 1;
      right = right > 0 ? right : 0;
      on = kvh < sparse_heads ? ((left + right) % p.vert_stride == 0) : true;
    }
    if (p.causal) on = on && (qp >= kp);  // dkernel/utils.py:213-215
    mask[i] = on ? 1 : 0;
  }
}

// One warp per (row, head): number of non-zeros -> crow[h][m+1].
__global__ void row_count_kernel(const uint8_t* __restrict__ mask, int H, int M, int N,
                                 int64_t sh, int64_t sm, int64_t sn, int32_t* __restrict__ crow) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (row >= (long long)H * M) return;
  const int h = (int)(row / M), m = (int)(row % M);
  const uint8_t* base = mask + h * sh + m * sm;
  int cnt = 0;
  for (int n = lane; n < N; n += 32) cnt += base[n * sn] != 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if (lane == 0) crow[(long long)h * (M + 1) + m + 1] = cnt;
}

// One block per head: in-place inclusive scan of crow[h][1..M], crow[h][0] = 0.
__global__ void row_scan_kernel(int M, int32_t* __restrict__ crow, int32_t* __restrict__ nnz) {
  __shared__ int warp_sums[32];
  __shared__ int carry_s;
  int32_t* c = crow + (long long)blockIdx.x * (M + 1);
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  if (tid == 0) { c[0] = 0; carry_s = 0; }
  __syncthreads();
  for (int base = 0; base < M; base += blockDim.x) {
    const int i = base + tid;
    int v = i < M ? c[i + 1] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += t;
    }
    if (lane == 31) warp_sums[wid] = v;
    __syncthreads();
    if (wid == 0) {
      int w = lane < (int)(blockDim.x >> 5) ? warp_sums[lane] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += t;
      }
      warp_sums[lane] = w;
    }
    __syncthreads();
    const int carry = carry_s;
    v += carry + (wid > 0 ? warp_sums[wid - 1] : 0);
    if (i < M) c[i + 1] = v;
    __syncthreads();
    if (tid == blockDim.x - 1) carry_s = v;
    __syncthreads();
  }
  if (tid == 0 && nnz) nnz[blockIdx.x] = c[M];
}

// One warp per (row, head) writes the ordered column indices of that row; rows
// m == M are virtual and write the -1 padding of the head.
__global__ void fill_cols_kernel(const uint8_t* __restrict__ mask, int H, int M, int N,
                                 int64_t sh, int64_t sm, int64_t sn,
                                 const int32_t* __restrict__ crow, int32_t* __restrict__ col,
                                 int width, int interleave) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (row >= (long long)H * (M + 1)) return;
  const int h = (int)(row / (M + 1)), m = (int)(row % (M + 1));
  const int32_t* c = crow + (long long)h * (M + 1);
  const int es = interleave ? 2 : 1;
  int32_t* out = col + (long long)h * width * es;
  if (m == M) {
    for (int i = c[M] + lane; i < width; i += 32) {
      out[i * es] = -1;
      if (interleave) out[i * es + 1] = 0;
    }
    return;
  }
  const uint8_t* base = mask + h * sh + m * sm;
  int pos = c[m];
  for (int n0 = 0; n0 < N; n0 += 32) {
    const int n = n0 + lane;
    const uint8_t val = n < N ? base[n * sn] : 0;
    const unsigned bal = __ballot_sync(0xffffffffu, val != 0);
    if (val != 0) {
      const int r = pos + __popc(bal & ((1u << lane) - 1u));
      if (r < width) {
        out[r * es] = n;
        if (interleave) out[r * es + 1] = val;
      }
    }
    pos += __popc(bal);
  }
}

}  // namespace

int layout_local_stride_mask(const bsa_local_stride_params* p, uint8_t* mask, cudaStream_t s) {
  BSA_CHECK_ARG(p && mask, "bsa_local_stride_mask: null argument");
  BSA_CHECK_ARG(p->num_heads >= 1 && p->num_kv_heads >= 1 && p->num_heads % p->num_kv_heads == 0,
                "bsa_local_stride_mask: num_heads=%d must be a multiple of num_kv_heads=%d",
                p->num_heads, p->num_kv_heads);
  BSA_CHECK_ARG(p->vert_stride >= 1, "bsa_local_stride_mask: vert_stride must be >= 1");
  BSA_CHECK_ARG(p->q_blocks >= 0 && p->kv_blocks >= 0 && p->trim_q_blocks >= 0,
                "bsa_local_stride_mask: negative size");
  const int rows = p->q_blocks - p->trim_q_blocks;
  const long long total = rows <= 0 ? 0 : (long long)p->num_heads * rows * p->kv_blocks;
  if (total == 0) return BSA_OK;
  const int threads = 256;
  long long blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  local_stride_mask_kernel<<<(unsigned)blocks, threads, 0, s>>>(*p, mask);
  return check_launch("local_stride_mask_kernel");
}

int layout_csr_row_ptr(const uint8_t* mask, int H, int M, int N, int64_t sh, int64_t sm, int64_t sn,
                       int32_t* crow, int32_t* nnz, cudaStream_t s) {
  BSA_CHECK_ARG(crow && (mask || (long long)H * M * N == 0), "bsa_csr_row_ptr: null argument");
  BSA_CHECK_ARG(H >= 1 && M >= 0 && N >= 0, "bsa_csr_row_ptr: bad shape (%d,%d,%d)", H, M, N);
  if (M > 0) {
    const long long rows = (long long)H * M;
    row_count_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(mask, H, M, N, sh, sm, sn, crow);
    int rc = check_launch("row_count_kernel");
    if (rc) return rc;
  }
  row_scan_kernel<<<H, 1024, 0, s>>>(M, crow, nnz);
  return check_launch("row_scan_kernel");
}

int layout_csr_fill_cols(const uint8_t* mask, int H, int M, int N, int64_t sh, int64_t sm, int64_t sn,
                         const int32_t* crow, int32_t* col, int width, int interleave,
                         cudaStream_t s) {
  BSA_CHECK_ARG(crow && (col || width == 0), "bsa_csr_fill_cols: null argument");
  BSA_CHECK_ARG(H >= 1 && M >= 0 && N >= 0 && width >= 0, "bsa_csr_fill_cols: bad shape");
  if (width == 0) return BSA_OK;
  const long long rows = (long long)H * (M + 1);
  fill_cols_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(mask, H, M, N, sh, sm, sn, crow, col,
                                                             width, interleave);
  return check_launch("fill_cols_kernel");
}

}  // namespace bsa
