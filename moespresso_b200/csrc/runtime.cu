// Host-side plumbing shared by every entry point: error strings, device
// properties, TMA descriptor encoding.
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include <atomic>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace mxb {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tensor_map(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return fail(MXB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bx[5];
  cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i - 1];
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
    return fail(MXB_ERR_INVALID, "tensor base address must be 16-byte aligned for TMA");
  for (int i = 0; i + 1 < rank; ++i)
    if (gstr[i] % 16 != 0) return fail(MXB_ERR_INVALID, "tensor strides must be multiples of 16 bytes for TMA");
  CUresult r = enc(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bx, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MXB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return MXB_OK;
}

}  // namespace mxb

namespace mxb {
static std::atomic<long long> g_launches{0};
void note_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
}  // namespace mxb

extern "C" int64_t mxb_kernel_launches(void) { return mxb::g_launches.load(std::memory_order_relaxed); }
extern "C" int mxb_copy_h2d_async(void* dst_device, const void* src_host, int64_t bytes, void* stream) {
  MXB_REQUIRE(dst_device && src_host && bytes >= 0, MXB_ERR_INVALID, "copy: null pointer or negative size");
  MXB_CUDA_OK(cudaMemcpyAsync(dst_device, src_host, (size_t)bytes, cudaMemcpyHostToDevice,
                              reinterpret_cast<cudaStream_t>(stream)));
  return MXB_OK;
}

namespace mxb {
__global__ void range_candidates_kernel(mxb_range_candidates_args a) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= a.k) return;
  const int32_t id = a.ids[i];
  a.out_scores[i] = id >= 0 ? a.scores[id] : -INFINITY;
  a.out_ids[i] = id >= 0 ? (int32_t)(id + a.row_lo) : -1;
}
__global__ void range_local_ids_kernel(mxb_range_local_ids_args a) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= a.k) return;
  const int32_t pos = a.pos[i];
  int64_t g = -1;
  if (pos >= 0) g = a.cand_ids[(int64_t)(pos / a.k) * a.cand_rank_stride + pos % a.k];
  a.out[i] = (g >= a.row_lo && g < a.row_lo + a.rows_local) ? (int32_t)(g - a.row_lo) : -1;
}
}  // namespace mxb

extern "C" int mxb_range_candidates(const mxb_range_candidates_args* a, void* stream) {
  MXB_REQUIRE(a != nullptr && a->k > 0, MXB_ERR_INVALID, "range candidates: null args or empty list");
  MXB_REQUIRE(a->scores && a->ids && a->out_scores && a->out_ids, MXB_ERR_INVALID, "range candidates: null tensor");
  MXB_REQUIRE(a->row_lo >= 0 && a->row_lo < ((int64_t)1 << 31), MXB_ERR_INVALID, "range candidates: global ids must fit 31 bits");
  mxb::range_candidates_kernel<<<(a->k + 255) / 256, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*a);
  mxb::note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}

extern "C" int mxb_range_local_ids(const mxb_range_local_ids_args* a, void* stream) {
  MXB_REQUIRE(a != nullptr && a->k > 0, MXB_ERR_INVALID, "range local ids: null args or empty list");
  MXB_REQUIRE(a->pos && a->cand_ids && a->out, MXB_ERR_INVALID, "range local ids: null tensor");
  MXB_REQUIRE(a->rows_local >= 0 && a->row_lo >= 0, MXB_ERR_INVALID, "range local ids: negative row range");
  mxb::range_local_ids_kernel<<<(a->k + 255) / 256, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*a);
  mxb::note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}

extern "C" int mxb_abi_version(void) { return MXB_ABI_VERSION; }
extern "C" const char* mxb_last_error(void) { return mxb::g_err; }
