// Host runtime shared by all kernels: per-device status words, tensor-map encoding through
// the driver entry point (no link-time dependency on libcuda), device properties.
#include "common.cuh"

#include <string.h>

__device__ int xb_status_words_dev[8];

namespace {
std::mutex g_mu;
int* g_status_ptr[64] = {nullptr};
int g_sm_count[64] = {0};
xb_encode_tiled_fn g_encode = nullptr;
}  // namespace

int* xb_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_status_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, xb_status_words_dev) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 8 * sizeof(int));
    g_status_ptr[dev] = (int*)p;
  }
  return g_status_ptr[dev];
}

int xb_sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_sm_count[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    g_sm_count[dev] = n > 0 ? n : 148;
  }
  return g_sm_count[dev];
}

xb_encode_tiled_fn xb_get_encode_tiled() {
  // The driver entry point needs a CUDA context bound to the calling thread.  A fresh thread whose
  // device is 0 (e.g. an autograd worker) has none until its first runtime call, so make one.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(0);
    ctx_bound = true;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) !=
            cudaSuccess ||
        qres != cudaDriverEntryPointSuccess) {
      return nullptr;
    }
    g_encode = (xb_encode_tiled_fn)fn;
  }
  return g_encode;
}

int xb_make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_size,
                    uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                    uint32_t box_cols, CUtensorMapSwizzle swz) {
  xb_encode_tiled_fn enc = xb_get_encode_tiled();
  if (!enc) return -1;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstr[1] = {ld * (uint64_t)elem_size};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr, "xb_make_tmap_2d failed (%d): base=%p rows=%llu cols=%llu ld=%llu box=%ux%u es=%d\n",
            (int)r, base, (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld,
            box_rows, box_cols, elem_size);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

int xb_make_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_size,
                    uint64_t batch, uint64_t rows, uint64_t cols, uint64_t ld_batch,
                    uint64_t ld_row, uint32_t box_batch, uint32_t box_rows, uint32_t box_cols,
                    CUtensorMapSwizzle swz) {
  xb_encode_tiled_fn enc = xb_get_encode_tiled();
  if (!enc) return -1;
  cuuint64_t gdim[3] = {cols, rows, batch};
  cuuint64_t gstr[2] = {ld_row * (uint64_t)elem_size, ld_batch * (uint64_t)elem_size};
  cuuint32_t box[3] = {box_cols, box_rows, box_batch};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, dt, 3, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// Reads and clears the calling device's status words.  out[0] != 0 means a kernel gave up on
// a bounded wait (or rejected its arguments) since the last call.  Synchronises the device.
XB_API int xb_status_read(int* out8, int clear) {
  int* p = xb_status_ptr();
  if (!p) return -1;
  if (cudaMemcpy(out8, p, 8 * sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (clear) cudaMemset(p, 0, 8 * sizeof(int));
  return 0;
}

XB_API int xb_device_sm_count() { return xb_sm_count(); }

XB_API const char* xb_build_info() { return "xorl_b200 csrc sm_100a"; }
