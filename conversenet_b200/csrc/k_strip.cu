// Multi-pass (strip) kernels for planes that do not fit in shared memory: three
// launches per chunk of plane pairs, meeting in the caller's workspace.
#include "../../include/converse_b200.h"
#include "cvb_internal.h"
#include "cvb_strip.cuh"
#include "cvb_plan.h"

namespace cvb {

constexpr int kStripThreads = 256;

template <typename IO>
__global__ void __launch_bounds__(kStripThreads, 2) strip_colfwd_kernel(const StripParams SP) {
  extern __shared__ float2 smem[];
  strip_colfwd_body<IO>(SP, blockIdx.y, blockIdx.x, smem, 0);
}
__global__ void __launch_bounds__(kStripThreads, 2) strip_rowmid_kernel(const StripParams SP) {
  extern __shared__ float2 smem[];
  strip_rowmid_body(SP, blockIdx.y, blockIdx.x, smem, 0);
}
template <typename IO>
__global__ void __launch_bounds__(kStripThreads, 2) strip_colinv_kernel(const StripParams SP) {
  extern __shared__ float2 smem[];
  strip_colinv_body<IO>(SP, blockIdx.y, blockIdx.x, smem, 0);
}

namespace {
template <typename IO>
int launch_t(const FwdParams& P, void* workspace, size_t ws_bytes, cudaStream_t st,
             size_t ws_cap = kWorkspaceTarget, bool at_least_one = true) {
  const int npairs = num_pairs(P);
  const StripGeo g = strip_geometry(P.h, P.w, P.k, P.s, npairs, ws_cap, at_least_one);
  if (g.chunk_pairs < 1) return CVB_ERR_TOO_LARGE;
  if (!workspace || ws_bytes < g.ws_bytes) return CVB_ERR_WORKSPACE;
  if (g.smem_col > kSmemLimit || g.smem_row > kSmemLimit) return CVB_ERR_UNSUPPORTED_SIZE;
  CVB_CUDA(cudaFuncSetAttribute(strip_colfwd_kernel<IO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem_col));
  CVB_CUDA(cudaFuncSetAttribute(strip_colinv_kernel<IO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem_col));
  CVB_CUDA(cudaFuncSetAttribute(strip_rowmid_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem_row));
  StripParams SP;
  SP.f = P;
  SP.ws = (float2*)workspace;
  SP.cw = g.cw; SP.rh = g.rh; SP.halo_l = g.halo_l; SP.halo_r = g.halo_r;
  const int ncs = (P.w + g.cw - 1) / g.cw, nrs = (P.h + g.rh - 1) / g.rh;
  for (int p0 = 0; p0 < npairs; p0 += g.chunk_pairs) {
    SP.pair0 = p0;
    SP.npair = (npairs - p0) < g.chunk_pairs ? (npairs - p0) : g.chunk_pairs;
    strip_colfwd_kernel<IO><<<dim3(ncs, SP.npair), kStripThreads, g.smem_col, st>>>(SP);
    strip_rowmid_kernel<<<dim3(nrs, SP.npair), kStripThreads, g.smem_row, st>>>(SP);
    strip_colinv_kernel<IO><<<dim3(ncs, SP.npair), kStripThreads, g.smem_col, st>>>(SP);
    CVB_CUDA(cudaGetLastError());
  }
  return CVB_OK;
}
}  // namespace

// ---- scratch that nobody has to allocate -------------------------------------------
// Some callers of this library cannot call cudaMalloc (or any allocator) at the point
// where they run the operator: code inside a stream-ordered region whose memory pool is
// frozen, a plug-in that was handed only its input and output buffers, a latency-critical
// loop that must not touch the allocator lock.  For them the workspace of the multi-pass
// path lives here, in the library image: every GPU that loads the library holds these
// CVB_STATIC_SCRATCH_BYTES until the process exits.
//
// In host code `g_static_scratch` is only a handle for the runtime, not a device
// address; the address a kernel may use comes from cudaGetSymbolAddress, asked once per
// device with that device current.
static __device__ __align__(256) unsigned char g_static_scratch[CVB_STATIC_SCRATCH_BYTES];

static int static_scratch_address(void** out) {
  static void* ptrs[64] = {nullptr};
  int dev = 0;
  CVB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return CVB_ERR_BAD_ARGUMENT;
  if (!ptrs[dev]) {
    void* p = nullptr;
    CVB_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return CVB_OK;
}

int launch_strip_static_scratch(const FwdParams& P, int io_dtype, cudaStream_t st) {
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != CVB_OK) return rc;
  // the chunk of plane pairs is sized to the fixed array; a plane pair that does not fit is refused
  return io_dtype == CVB_F32
             ? launch_t<float>(P, scratch, CVB_STATIC_SCRATCH_BYTES, st, CVB_STATIC_SCRATCH_BYTES, false)
             : launch_t<__nv_bfloat16>(P, scratch, CVB_STATIC_SCRATCH_BYTES, st, CVB_STATIC_SCRATCH_BYTES, false);
}

int launch_strip(const FwdParams& P, int io_dtype, void* workspace, size_t ws_bytes, cudaStream_t st) {
  return io_dtype == CVB_F32 ? launch_t<float>(P, workspace, ws_bytes, st)
                             : launch_t<__nv_bfloat16>(P, workspace, ws_bytes, st);
}

}  // namespace cvb
