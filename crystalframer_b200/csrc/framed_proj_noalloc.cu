// cfb200_framed_proj_bwd_noalloc: the backward pass of the lattice-sum bias / value encoding for
// hosts that cannot give the library scratch memory.
//
// The regular entry point, cfb200_framed_proj_bwd, needs a caller-provided workspace (per-pair
// coefficient gradients and per-block weight-gradient partials).  Some hosts have nowhere to take
// it from: a plugin that runs under a runtime owning the whole device heap and is handed only its
// input and output buffers, or a service whose rules forbid device allocation once it has started
// (cudaMalloc synchronises the device and may fail on a fragmented heap).  For them the scratch
// lives in the fixed-size device array below.  The price: every process that loads the library
// holds kNoAllocBytes of device memory on each GPU it touches until it exits, and problem sizes
// whose scratch need exceeds that are refused.
//
// This file is included at the end of api.cu (the library is one translation unit).
#include <mutex>

namespace cfb_noalloc {

constexpr size_t kNoAllocBytes = (size_t)CFB200_NOALLOC_MAX_BYTES;

// File-scope device array.  In host code this name is only a handle for the runtime, not a
// device address: the address is obtained once per device with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_scratch[kNoAllocBytes];

static std::mutex g_mutex;
static void* g_scratch_ptr[64] = {nullptr};

// Device address of the scratch array on the current device, resolved on first use.
static int scratch_address(void** out)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return CFB200_E_CUDA;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_scratch) != cudaSuccess || p == nullptr) return CFB200_E_CUDA;
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return CFB200_OK;
}

}  // namespace cfb_noalloc

extern "C" int cfb200_framed_proj_bwd_noalloc(
    const float* a_ik, const float* pos_ij, const float* tvecs, const float* rvlen, const int64_t* batch,
    const int64_t* edges, const int64_t* e_start, int64_t N, int64_t E, float dist_max, float cutoff_radius,
    const float* W_dist, const float* W_ang1, const float* W_ang2, const float* W_ang3, const float* frame1,
    const float* frame2, const float* frame3, const float* z, const float* gz, const float* gvalues, float* ga,
    float* gW_dist, float* gW_ang1, float* gW_ang2, float* gW_ang3, void* stream)
{
    const int64_t need = cfb200_framed_proj_bwd_workspace_bytes(N, E);
    if (need < 0) return N < 0 || E < 0 ? CFB200_E_SHAPE : CFB200_E_NOT_CONFIGURED;
    if ((size_t)need > cfb_noalloc::kNoAllocBytes) return CFB200_E_TOO_LARGE;
    void* scratch = nullptr;
    const int rc = cfb_noalloc::scratch_address(&scratch);
    if (rc != CFB200_OK) return rc;
    // Both scratch regions are fully overwritten by the kernels before they are read, so the
    // contents the previous call left behind need no clearing.
    return cfb200_framed_proj_bwd(a_ik, pos_ij, tvecs, rvlen, batch, edges, e_start, N, E, dist_max, cutoff_radius,
                                  W_dist, W_ang1, W_ang2, W_ang3, frame1, frame2, frame3, z, gz, gvalues, ga, gW_dist,
                                  gW_ang1, gW_ang2, gW_ang3, scratch, (int64_t)cfb_noalloc::kNoAllocBytes, stream);
}
