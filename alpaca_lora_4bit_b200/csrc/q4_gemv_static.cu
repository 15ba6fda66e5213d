// q4_gemv_static: the decode product for callers that must not allocate device memory.
//
// Some hosts of this library cannot hand it a workspace: an inference server that gave every byte
// of HBM to its own pools at start-up, a plugin loaded into a process whose allocator it may not
// touch, or code on a latency path where cudaMalloc (which synchronises the device) is off limits.
// For them the scratch that q4_gemv normally receives from the caller lives here, in a file-scope
// device array that every GPU loading the library carries until the process exits.
#include <mutex>

#include "q4_common.cuh"

namespace q4 {

constexpr size_t GEMV_STATIC_SCRATCH_BYTES = 131072 + (2u << 20);    // 2.125 MiB per device: what every
                                                                    // sequential-group shape needs

static __device__ __align__(256) unsigned char g_gemv_static_scratch[GEMV_STATIC_SCRATCH_BYTES];

// In host code the array's name is only a handle; the device address of each GPU's copy has to be
// asked for, once per device and with that device current.
static void* g_scratch_ptr[64] = {nullptr};
static std::mutex g_scratch_mutex;

static int static_scratch(void** out) {
  int dev = 0;
  if (int e = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return e;
  if (dev < 0 || dev >= 64) return fail(Q4_E_DEVICE, "gemv_static: device index %d not supported", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    if (int e = check_cuda(cudaGetSymbolAddress(&p, g_gemv_static_scratch), "cudaGetSymbolAddress(scratch)")) return e;
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return Q4_OK;
}

}  // namespace q4

using namespace q4;

extern "C" size_t q4_gemv_static_max_bytes(void) { return GEMV_STATIC_SCRATCH_BYTES; }

extern "C" int q4_gemv_static(const void* x, const int32_t* qweight, void* y, const void* scales,
                              const int32_t* qzeros, const int32_t* g_idx, const void* bias,
                              int M, int K, int N, int G, int groupsize, int y_dtype, unsigned flags,
                              q4_stream_t stream) {
  const size_t need = q4_gemv_workspace_bytes(M, K, N);
  if (need == 0) return fail(Q4_E_SHAPE, "gemv_static: M=%d K=%d N=%d not supported (K, N multiples of 32)", M, K, N);
  if (need > GEMV_STATIC_SCRATCH_BYTES)
    return fail(Q4_E_WORKSPACE, "gemv_static: this shape needs %zu bytes of scratch, the built-in scratch holds %zu; "
                "use q4_gemv with a caller-provided workspace", need, (size_t)GEMV_STATIC_SCRATCH_BYTES);
  void* scratch = nullptr;
  if (int e = static_scratch(&scratch)) return e;
  // The array keeps whatever the previous call left.  The kernels need the arrival counters at its head to
  // start at zero; a normal call leaves them so, one whose bounded wait expired may not.  The status word
  // (the last word of the head) is left alone: it stays set until q4_gemv_static_status has reported it.
  if (int e = check_cuda(cudaMemsetAsync(scratch, 0, 65536 - 4, (cudaStream_t)stream), "clear scratch head")) return e;
  if (int e = check_cuda(cudaMemsetAsync((char*)scratch + 65536, 0, 65536 - 4, (cudaStream_t)stream), "clear scratch head")) return e;
  return q4_gemv(x, qweight, y, scales, qzeros, g_idx, bias, M, K, N, G, groupsize, y_dtype, flags,
                 scratch, GEMV_STATIC_SCRATCH_BYTES, stream);
}

extern "C" int q4_gemv_static_status(unsigned* out) {
  if (!out) return fail(Q4_E_BADARG, "gemv_static_status: null pointer");
  void* scratch = nullptr;
  if (int e = static_scratch(&scratch)) return e;
  if (int e = q4_gemv_status(scratch, GEMV_STATIC_SCRATCH_BYTES, out)) return e;
  if (*out) return check_cuda(cudaMemset((char*)scratch + 65536 - 4, 0, 4), "clear decode status");
  return Q4_OK;
}
