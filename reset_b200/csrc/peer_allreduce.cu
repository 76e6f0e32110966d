// One-shot all-reduce of a small bf16 tensor over NVLink peer memory: the sum exchange after
// a row-parallel decode linear ([M, hidden] bf16: 10 KB at M = 1). One kernel per rank, no
// library call inside:
//   push    every thread packs two bf16 values with a flag into ONE 64-bit slot {1 : bf16x2}
//           and stores it into the receive area of every rank (its own included) with plain
//           peer stores; a 64-bit scalar store is single-copy atomic, so a slot is either
//           still zero or complete (no fence, no separate flag);
//   gather  the same thread polls its slot in each of the W receive rows of ITS OWN memory,
//           adds the W values in rank order in fp32 (every rank computes the same bits),
//           rounds once to bf16, and writes zeros back into the slots it consumed.
// The receive area is double-buffered by call parity. A rank can be at most one call ahead of
// a peer (it cannot finish call n+1 before the peer has pushed call n+1, which the peer does
// only after finishing call n), so the slots of parity p are always consumed and zeroed
// before anyone pushes into them again. The parity comes from a call counter in the rank's
// own memory that the last CTA of every launch advances, so a captured CUDA graph can be
// replayed any number of times.
// Nothing here uses multicast loads or TMA on peer memory: pushes are ordinary st.global to
// a peer pointer, polls are ordinary loads of local memory. Polls are bounded; on expiry the
// kernel sets the status word read by nvfp4r_check_device_status and returns.
#include <cuda_bf16.h>

#include <cstring>

#include "../../include/nvfp4r_b200.h"
#include "kernels.h"
#include "status_mirror.cuh"
#include "nvfp4_ptx.cuh"

namespace nvfp4r {
namespace {

constexpr int kMaxWorld = NVFP4R_PEER_MAX_WORLD;
constexpr size_t kHeaderBytes = 256;                 // [0] call counter, [1] finished-CTA counter
constexpr uint32_t kPeerPollLimit = 4000000u;        // default: a second or two; a dead peer ends the wait, not the GPU
uint32_t g_peer_poll_limit = kPeerPollLimit;         // host copy, passed with every launch

__device__ int g_peer_status = 0;

struct PeerParams {
    unsigned char* base[kMaxWorld];                  // receive memory of every rank (own: local pointer)
    int world, rank;
    unsigned long long max_pairs;                    // slots per (parity, source rank) row
    const uint32_t* in;                              // bf16x2 words
    uint32_t* out;
    unsigned long long pairs;
    int mode;                                        // bit 0: push, bit 1: gather
    uint32_t poll_limit;
};

__device__ __forceinline__ void peer_store(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" :: "l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long local_poll(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(256)
peer_allreduce_kernel(const PeerParams p) {
    __shared__ int s_failed;
    if (threadIdx.x == 0) s_failed = 0;
    pdl_launch_dependents();
    pdl_wait_prior();                                // the input is the previous kernel's output
    unsigned* header = reinterpret_cast<unsigned*>(p.base[p.rank]);
    const unsigned parity = *reinterpret_cast<volatile unsigned*>(header) & 1u;
    __syncthreads();
    const unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const unsigned long long row = p.max_pairs;
    if (i < p.pairs) {
        if (p.mode & 1) {
            const unsigned long long w = (1ull << 32) | static_cast<unsigned long long>(p.in[i]);
#pragma unroll 1
            for (int d = 0; d < p.world; ++d) {
                const int dst = (p.rank + d) % p.world;      // spread the first stores over the links
                unsigned long long* slots = reinterpret_cast<unsigned long long*>(p.base[dst] + kHeaderBytes);
                peer_store(slots + (static_cast<unsigned long long>(parity) * p.world + p.rank) * row + i, w);
            }
        }
        if (p.mode & 2) {
            unsigned long long* mine = reinterpret_cast<unsigned long long*>(p.base[p.rank] + kHeaderBytes) +
                                       static_cast<unsigned long long>(parity) * p.world * row + i;
            unsigned long long v[kMaxWorld];
#pragma unroll
            for (int s = 0; s < kMaxWorld; ++s)
                if (s < p.world) v[s] = local_poll(mine + s * row);
            bool ok = true;
            for (uint32_t it = 0;; ++it) {
                bool all = true;
#pragma unroll
                for (int s = 0; s < kMaxWorld; ++s)
                    if (s < p.world && (v[s] >> 32) != 1ull) {
                        v[s] = local_poll(mine + s * row);
                        all = false;
                    }
                if (all) break;
                if (it > p.poll_limit) { ok = false; break; }
            }
            float lo = 0.0f, hi = 0.0f;
#pragma unroll
            for (int s = 0; s < kMaxWorld; ++s)
                if (s < p.world) {
                    const uint32_t w = static_cast<uint32_t>(v[s]);
                    lo += __uint_as_float(w << 16);
                    hi += __uint_as_float(w & 0xFFFF0000u);
                    mine[s * row] = 0ull;
                }
            const __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
            p.out[i] = *reinterpret_cast<const uint32_t*>(&r);
            if (!ok) s_failed = 1;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (s_failed) report_timeout(&g_peer_status, 4);
        if (p.mode & 2) {
            // the last CTA to finish advances the call counter: nobody of this launch reads it any more
            __threadfence();
            const unsigned t = atomicAdd(header + 1, 1u);
            if (t == gridDim.x - 1) {
                header[1] = 0u;
                header[0] = header[0] + 1u;
            }
        }
    }
}

}  // namespace

uint32_t peer_poll_limit() { return g_peer_poll_limit; }

cudaError_t set_status_mirror_peer(int* p) { return set_status_mirror_here(p); }

cudaError_t read_and_clear_peer_status(int* flag) {
    cudaError_t e = cudaMemcpyFromSymbol(flag, g_peer_status, sizeof(int));
    if (e != cudaSuccess) return e;
    const int zero = 0;
    return cudaMemcpyToSymbol(g_peer_status, &zero, sizeof(int));
}

}  // namespace nvfp4r

using namespace nvfp4r;

extern "C" {

size_t nvfp4r_peer_buffer_bytes(int world, size_t max_elems) {
    if (world < 1 || world > kMaxWorld || max_elems == 0) return 0;
    const size_t pairs = (max_elems + 1) / 2;
    return kHeaderBytes + 2 * static_cast<size_t>(world) * pairs * sizeof(unsigned long long);
}

int nvfp4r_peer_alloc(size_t bytes, void** ptr, unsigned char* handle64) {
    if (!ptr || !handle64 || bytes == 0) return NVFP4R_ERR_INVALID_ARGUMENT;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) return NVFP4R_ERR_CUDA;
    if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) { cudaFree(p); return NVFP4R_ERR_CUDA; }
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) { cudaFree(p); return NVFP4R_ERR_CUDA; }
    memcpy(handle64, &h, 64);
    *ptr = p;
    return NVFP4R_OK;
}

int nvfp4r_peer_open(const unsigned char* handle64, void** peer_ptr) {
    if (!handle64 || !peer_ptr) return NVFP4R_ERR_INVALID_ARGUMENT;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return NVFP4R_ERR_CUDA;
    *peer_ptr = p;
    return NVFP4R_OK;
}

int nvfp4r_peer_close(void* peer_ptr) {
    if (!peer_ptr) return NVFP4R_ERR_INVALID_ARGUMENT;
    return cudaIpcCloseMemHandle(peer_ptr) == cudaSuccess ? NVFP4R_OK : NVFP4R_ERR_CUDA;
}

int nvfp4r_peer_free(void* ptr) {
    if (!ptr) return NVFP4R_ERR_INVALID_ARGUMENT;
    return cudaFree(ptr) == cudaSuccess ? NVFP4R_OK : NVFP4R_ERR_CUDA;
}

int nvfp4r_set_peer_poll_limit(unsigned polls) {
    g_peer_poll_limit = polls == 0 ? kPeerPollLimit : polls;
    return NVFP4R_OK;
}

int nvfp4r_peer_allreduce_bf16(const nvfp4r_peer_comm* comm, const void* in, void* out, size_t count,
                               int mode, void* stream) {
    if (!comm || !in || !out || count == 0 || (count & 1)) return NVFP4R_ERR_INVALID_ARGUMENT;
    if (comm->world < 1 || comm->world > kMaxWorld || comm->rank < 0 || comm->rank >= comm->world)
        return NVFP4R_ERR_INVALID_ARGUMENT;
    if (mode < 1 || mode > 3) return NVFP4R_ERR_INVALID_ARGUMENT;
    const size_t pairs = count / 2, max_pairs = (comm->max_elems + 1) / 2;
    if (pairs > max_pairs) return NVFP4R_ERR_UNSUPPORTED_SHAPE;
    if ((reinterpret_cast<uintptr_t>(in) & 3) || (reinterpret_cast<uintptr_t>(out) & 3)) return NVFP4R_ERR_INVALID_ARGUMENT;
    PeerParams p = {};
    for (int r = 0; r < comm->world; ++r) {
        if (!comm->base[r]) return NVFP4R_ERR_INVALID_ARGUMENT;
        p.base[r] = static_cast<unsigned char*>(comm->base[r]);
    }
    p.world = comm->world;
    p.rank = comm->rank;
    p.max_pairs = max_pairs;
    p.in = static_cast<const uint32_t*>(in);
    p.out = static_cast<uint32_t*>(out);
    p.pairs = pairs;
    p.mode = mode;
    p.poll_limit = g_peer_poll_limit;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>((pairs + 255) / 256));
    cfg.blockDim = dim3(256);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = gemv_tuning().use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, peer_allreduce_kernel, p) == cudaSuccess ? NVFP4R_OK : NVFP4R_ERR_CUDA;
}

}  // extern "C"
