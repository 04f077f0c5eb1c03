// Host side of TMA: tensor-map encoding through the driver entry point (no
// link-time dependency on libcuda, so the library also loads on a machine
// without a driver) and the thread-local error text.
#include <climits>
#include <mutex>

#include "ptx.cuh"

namespace bsa {

namespace {
thread_local char g_err[512] = "";
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
const char* last_error() { return g_err; }

static PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault,
                                         &qr) == cudaSuccess &&
        qr == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

bool tma_compatible(const void* base, int elem_bytes, int64_t ss, int64_t sh, int64_t sb) {
  if (reinterpret_cast<uintptr_t>(base) % 16) return false;
  const int64_t m = 16 / elem_bytes;
  return ss > 0 && sh >= 0 && sb >= 0 && ss % m == 0 && sh % m == 0 && sb % m == 0;
}

int make_tmap_4d(Tmap4* out, const void* base, int elem_bytes, uint64_t d, uint64_t seq,
                 uint64_t heads, uint64_t batch, int64_t seq_stride_b, int64_t head_stride_b,
                 int64_t batch_stride_b, uint32_t box_d, uint32_t box_seq, bool swizzle128,
                 bool is_bf16) {
  auto enc = get_encode();
  if (!enc) {
    set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    return BSA_E_CUDA;
  }
  // The encoder is a driver entry point and wants a context current on the calling thread.  A
  // thread that has not made a runtime call yet (an autograd worker entering the backward, a
  // host's worker thread) has none: binding the device's primary context once per thread costs
  // nothing afterwards.
  thread_local bool context_bound = false;
  if (!context_bound) {
    if (cudaFree(nullptr) == cudaSuccess) context_bound = true;
    else (void)cudaGetLastError();   // e.g. refused during stream capture: the encode below decides
  }
  // The three outer dimensions are placed in order of increasing stride, so the
  // map looks like an ordinary padded row-major tensor whatever the caller's
  // layout ((B,S,H,D), (B,H,S,D), packed (T,H,D), views of larger tensors).
  // Dimensions of extent 1 (their stride is irrelevant, possibly 0) go last.
  struct Dim { uint64_t extent; int64_t stride; int logical; uint32_t box; };
  out->head_bcast = (heads <= 1 || head_stride_b <= 0) ? 1 : 0;
  out->batch_bcast = (batch <= 1 || batch_stride_b <= 0) ? 1 : 0;
  Dim dims3[3] = {{seq ? seq : 1, seq_stride_b, 0, box_seq},
                  {out->head_bcast ? 1 : heads, head_stride_b, 1, 1},
                  {out->batch_bcast ? 1 : batch, batch_stride_b, 2, 1}};
  auto key = [](const Dim& x) { return x.extent <= 1 ? INT64_MAX : x.stride; };
  for (int i = 0; i < 3; ++i)
    for (int j = i + 1; j < 3; ++j)
      if (key(dims3[j]) < key(dims3[i])) { Dim t = dims3[i]; dims3[i] = dims3[j]; dims3[j] = t; }
  cuuint64_t gdim[4] = {d, dims3[0].extent, dims3[1].extent, dims3[2].extent};
  cuuint64_t gstr[3];
  cuuint64_t prev = (cuuint64_t)(d * elem_bytes + 15) / 16 * 16;
  cuuint64_t prev_extent = 1;
  for (int i = 0; i < 3; ++i) {
    if (dims3[i].extent <= 1 || dims3[i].stride <= 0)
      gstr[i] = prev * prev_extent;  // any legal value: the coordinate is always 0
    else
      gstr[i] = (cuuint64_t)dims3[i].stride;
    prev = gstr[i];
    prev_extent = dims3[i].extent;
  }
  cuuint32_t box[4] = {box_d, dims3[0].box, dims3[1].box, dims3[2].box};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  for (int i = 0; i < 3; ++i) {
    if (dims3[i].logical == 0) out->seq_pos = i + 1;
    if (dims3[i].logical == 1) out->head_pos = i + 1;
    if (dims3[i].logical == 2) out->batch_pos = i + 1;
  }
  CUtensorMapDataType dt = elem_bytes == 4   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                           : elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                           : is_bf16         ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                             : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = enc(&out->map, dt, 4, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (dims %llu,%llu,%llu,%llu strides "
              "%llu,%llu,%llu box %u,%u,%u,%u)",
              (int)r, (unsigned long long)gdim[0], (unsigned long long)gdim[1],
              (unsigned long long)gdim[2], (unsigned long long)gdim[3],
              (unsigned long long)gstr[0], (unsigned long long)gstr[1],
              (unsigned long long)gstr[2], box[0], box[1], box[2], box[3]);
    return BSA_E_CUDA;
  }
  return BSA_OK;
}

}  // namespace bsa
