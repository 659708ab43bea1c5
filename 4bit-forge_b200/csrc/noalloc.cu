// Allocation-free factorisation of ONE Hessian.
//
// forge_chol_inv_upper_batched needs a caller-provided workspace (the inverted 64x64 diagonal blocks).
// Some callers cannot produce one at the moment they need a factorisation:
//   * the layer driver sizes its Hessian / factor batches to fill the GPU (a DeepSeek-V3-shaped layer
//     keeps > 100 GB of fp32 Hessians resident), so when one expert comes back with info > 0 and has
//     to be factorised again with a larger damping, there may be no free memory left to ask for;
//   * a host application that embeds the library under its own memory manager (a serving process
//     that partitions HBM among tenants at start-up, a framework allocator that must not be re-entered
//     from a callback) is not allowed to call cudaMalloc at all, and cudaMalloc would also synchronise
//     the device under the other streams.
// For them the workspace lives here, in a file-scope __device__ array that every GPU loading the
// library holds until the process exits (3 MiB for kMaxC = 4096: kMaxC^2/32 floats of inverted diagonal blocks and
// one inverted 512-column outer block).
//
// Rules of use (also in include/forge_b200.h):
//   * C <= FORGE_NOALLOC_MAX_C, otherwise FORGE_ERR_UNSUPPORTED;
//   * the first call on a device resolves the array's device address (cudaGetSymbolAddress, with that
//     device current); make that first call outside of any stream capture;
//   * all calls on a device share the one array: two calls whose kernels overlap on the GPU (different
//     streams) race.  Calls on one stream are ordered and safe.  Nothing in the array has to start at
//     zero — every block is written by the factorisation before it is read — so stale contents of an
//     earlier call are harmless.
#include "common.cuh"
#include <mutex>

using namespace forge;

namespace {

constexpr int64_t kMaxC = 4096;
// what forge_chol_workspace_bytes(1, kMaxC) asks for: one (Dinv, Dinv^T) pair per 64-column block, one inverted outer
// block (512 x 512), and the 256-byte tail for the status word of the tensor-core kernels
constexpr int64_t kScratchFloats = (kMaxC / 64) * 2 * 64 * 64 + 512 * 512 + 64;

// In host code this name is only a handle for the runtime, not a device address: the address the
// kernels can use comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_chol_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
float *g_scratch_ptr[kMaxDevices] = {nullptr};

// Once per device, with that device current.
int scratch_for_current_device(float **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_error("forge_chol_inv_upper_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
        return FORGE_ERR_LAUNCH;
    }
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_scratch_ptr[dev] == nullptr) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_chol_scratch);
        if (e != cudaSuccess || p == nullptr) {
            set_error("forge_chol_inv_upper_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            return FORGE_ERR_LAUNCH;
        }
        g_scratch_ptr[dev] = static_cast<float *>(p);
    }
    *out = g_scratch_ptr[dev];
    return FORGE_OK;
}

}  // namespace

extern "C" int64_t forge_noalloc_max_c(void) { return kMaxC; }

extern "C" int forge_chol_inv_upper_noalloc(float *A, int64_t C, float *U, float *udiag, int32_t *info,
                                            int zero_lower, void *stream) {
    FORGE_REQUIRE(A && U && udiag && info, "null pointer");
    FORGE_REQUIRE(C > 0, "empty matrix");
    if (C > kMaxC) {
        set_error("forge_chol_inv_upper_noalloc: C = %lld exceeds the built-in scratch (max C = %lld); "
                  "use forge_chol_inv_upper_batched with a caller workspace",
                  (long long)C, (long long)kMaxC);
        return FORGE_ERR_UNSUPPORTED;
    }
    float *scratch = nullptr;
    const int rc = scratch_for_current_device(&scratch);
    if (rc != FORGE_OK) return rc;
    // Same kernels, same order, same arithmetic as the batched entry point with a batch of one.
    return forge_chol_inv_upper_batched(A, 1, C, U, udiag, info, zero_lower, scratch, stream);
}
