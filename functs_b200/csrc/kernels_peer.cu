// Multi-GPU gather of the detection records without a collective library: the kernel that packs a rank's records
// stores them straight into every rank's gather buffer over NVLink (plain peer stores; the buffers are ordinary
// device allocations opened through CUDA IPC), followed by one flag per destination.
//
// Role in the sharded post-process: the reference runs one GPU; here a batch is split over the GPUs of a box and
// "only the final detections are gathered" - this file is that gather, fused with the packing of the records.
//
// Protocol (steps are numbered from 1; every rank owns a flag block of kPeerFlagWords words, zero at start):
//   arrived[src]  (in the destination's block)  last step whose records from rank src are complete there
//   consumed[dst] (in the writer's block)       last step whose gathered records rank dst has finished reading
//   writer, step s, slot s & 1:  wait consumed[dst] >= s - 2 for all dst  ->  store records to every dst
//                                -> fence -> the grid's last CTA sets arrived[me] = s at every dst
//   reader, step s:              peer_wait: arrived[src] >= s for all src; ... read ...; peer_release: consumed[me] = s
//                                at every src
// Every wait is bounded (about one second of clock cycles); when it runs out the kernel sets FB_STATUS_WAIT_TIMEOUT
// in the caller's status word and goes on without blocking, so a missing peer can never hang the GPU.
#include "common.cuh"

namespace fb {

constexpr int kPeerMaxRanks = 16;
constexpr int kPeerFlagWords = 64;  // [0,16) arrived, [16,32) consumed, [32] CTA ticket of the packing grid
constexpr unsigned long long kPeerWaitCycles = 2000000000ull;

struct PeerTable {
    int4* records[kPeerMaxRanks];      // every rank's gather buffer for this step's slot, [nranks * groups * topk * 2] int4
    uint32_t* flags[kPeerMaxRanks];    // every rank's flag block
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// waits until *p >= want (steps only grow); false when the bound ran out
__device__ __forceinline__ bool wait_flag_at_least(const uint32_t* p, uint32_t want) {
    const unsigned long long start = clock64();
    while (true) {
        if (static_cast<int32_t>(ld_acquire_sys(p) - want) >= 0) return true;
        if (clock64() - start > kPeerWaitCycles) return false;
        __nanosleep(200);
    }
}

__global__ void __launch_bounds__(256)
pack_store_peers_kernel(const float* __restrict__ dets, const int64_t* __restrict__ labels,
                        const int64_t* __restrict__ flat_ids, const int32_t* __restrict__ counts, int topk, int64_t total,
                        const PeerTable tab, int rank, int nranks, uint32_t step, int32_t* status) {
    __shared__ int s_last;
    uint32_t* mine = tab.flags[rank];
    // flow control: the slot may be overwritten once every destination has read what step - 2 left there
    if (threadIdx.x < nranks && step > 2u) {
        if (!wait_flag_at_least(mine + 16 + threadIdx.x, step - 2u) && status != nullptr) atomicOr(status, FB_STATUS_WAIT_TIMEOUT);
    }
    __syncthreads();
    const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i < total) {
        const int g = static_cast<int>(i / topk);
        const int k = static_cast<int>(i - static_cast<int64_t>(g) * topk);
        const float* d = dets + i * 5;
        int4 lo, hi;
        lo.x = __float_as_int(d[0]);
        lo.y = __float_as_int(d[1]);
        lo.z = __float_as_int(d[2]);
        lo.w = __float_as_int(d[3]);
        hi.x = __float_as_int(d[4]);
        hi.y = static_cast<int>(labels[i]);
        hi.z = static_cast<int>(flat_ids[i]);
        hi.w = k < counts[g] ? 1 : 0;
        const int64_t at = 2 * (static_cast<int64_t>(rank) * total + i);
        for (int r = 0; r < nranks; ++r) {
            int4* dst = tab.records[r] + at;
            dst[0] = lo;
            dst[1] = hi;
        }
    }
    // completion: all stores of this CTA are ordered before its ticket; the CTA that draws the last ticket tells
    // every destination that this rank's share of the step is there
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int t = atomicAdd(mine + 32, 1u);
        s_last = (t == gridDim.x - 1) ? 1 : 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence_system();
    if (threadIdx.x == 0) mine[32] = 0u;  // ready for the next launch (launches of one rank are stream-ordered)
    if (threadIdx.x < nranks) st_release_sys(tab.flags[threadIdx.x] + rank, step);
}

__global__ void peer_wait_kernel(const uint32_t* __restrict__ my_flags, int nranks, uint32_t step, int32_t* status) {
    if (threadIdx.x < nranks) {
        if (!wait_flag_at_least(my_flags + threadIdx.x, step) && status != nullptr) atomicOr(status, FB_STATUS_WAIT_TIMEOUT);
    }
}

__global__ void peer_release_kernel(const PeerTable tab, int rank, int nranks, uint32_t step) {
    if (threadIdx.x < nranks) st_release_sys(tab.flags[threadIdx.x] + 16 + rank, step);
}

static int fill_table(PeerTable& tab, void* const* records, void* const* flags, int nranks) {
    for (int r = 0; r < kPeerMaxRanks; ++r) {
        tab.records[r] = nullptr;
        tab.flags[r] = nullptr;
    }
    for (int r = 0; r < nranks; ++r) {
        if (flags[r] == nullptr || (records != nullptr && records[r] == nullptr)) return 1;
        tab.records[r] = records != nullptr ? static_cast<int4*>(records[r]) : nullptr;
        tab.flags[r] = static_cast<uint32_t*>(flags[r]);
    }
    return 0;
}

}  // namespace fb

extern "C" {

int32_t functs_b200_peer_flag_bytes(void) { return fb::kPeerFlagWords * 4; }

int functs_b200_peer_enable_access(int32_t peer_device) {
    using namespace fb;
    int dev = 0;
    FB_TRY(check_cuda(cudaGetDevice(&dev), "cudaGetDevice"));
    if (peer_device == dev) return FB_OK;
    int can = 0;
    FB_TRY(check_cuda(cudaDeviceCanAccessPeer(&can, dev, peer_device), "cudaDeviceCanAccessPeer"));
    FB_REQUIRE(can != 0, "peer_enable_access: device %d cannot reach device %d", dev, peer_device);
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();
        return FB_OK;
    }
    return check_cuda(e, "cudaDeviceEnablePeerAccess");
}

// Host-side look at a pointer that a kernel of the current device is about to use: it must be device memory, and
// if it lives on another GPU that GPU must be reachable (peer access is switched on here when it is not yet).
// Returns the owning device's ordinal in *device.
int functs_b200_peer_check_pointer(const void* ptr, int32_t* device) {
    using namespace fb;
    FB_REQUIRE(ptr != nullptr && device != nullptr, "peer_check_pointer: null pointer");
    cudaPointerAttributes at;
    FB_TRY(check_cuda(cudaPointerGetAttributes(&at, ptr), "cudaPointerGetAttributes"));
    FB_REQUIRE(at.type == cudaMemoryTypeDevice, "peer_check_pointer: %p is not device memory (type %d)", ptr,
               static_cast<int>(at.type));
    *device = at.device;
    return functs_b200_peer_enable_access(at.device);
}

int functs_b200_pack_detections_peers(const float* dets, const int64_t* labels, const int64_t* flat_ids,
                                      const int32_t* counts, int32_t groups, int32_t topk, void* const* peer_records,
                                      void* const* peer_flags, int32_t rank, int32_t nranks, uint32_t step,
                                      int32_t* status, void* stream) {
    using namespace fb;
    FB_REQUIRE(dets && labels && flat_ids && counts && peer_records && peer_flags, "pack_detections_peers: null pointer");
    FB_REQUIRE(groups > 0 && topk > 0 && nranks > 0 && nranks <= kPeerMaxRanks && rank >= 0 && rank < nranks && step > 0u,
               "pack_detections_peers: bad sizes (at most %d ranks, steps count from 1)", kPeerMaxRanks);
    PeerTable tab;
    FB_REQUIRE(fill_table(tab, peer_records, peer_flags, nranks) == 0, "pack_detections_peers: null peer pointer");
    for (int r = 0; r < nranks; ++r)
        FB_REQUIRE((reinterpret_cast<uintptr_t>(tab.records[r]) & 15) == 0, "pack_detections_peers: buffers must be 16-byte aligned");
    const int64_t total = static_cast<int64_t>(groups) * topk;
    pack_store_peers_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, as_stream(stream)>>>(
        dets, labels, flat_ids, counts, topk, total, tab, rank, nranks, step, status);
    count_launch();
    return check_launch("pack_store_peers_kernel");
}

int functs_b200_peer_wait(const void* my_flags, int32_t nranks, uint32_t step, int32_t* status, void* stream) {
    using namespace fb;
    FB_REQUIRE(my_flags != nullptr && nranks > 0 && nranks <= kPeerMaxRanks, "peer_wait: bad arguments");
    peer_wait_kernel<<<1, 32, 0, as_stream(stream)>>>(static_cast<const uint32_t*>(my_flags), nranks, step, status);
    count_launch();
    return check_launch("peer_wait_kernel");
}

int functs_b200_peer_release(void* const* peer_flags, int32_t rank, int32_t nranks, uint32_t step, void* stream) {
    using namespace fb;
    FB_REQUIRE(peer_flags != nullptr && nranks > 0 && nranks <= kPeerMaxRanks && rank >= 0 && rank < nranks,
               "peer_release: bad arguments");
    PeerTable tab;
    FB_REQUIRE(fill_table(tab, nullptr, peer_flags, nranks) == 0, "peer_release: null peer pointer");
    peer_release_kernel<<<1, 32, 0, as_stream(stream)>>>(tab, rank, nranks, step);
    count_launch();
    return check_launch("peer_release_kernel");
}

}  // extern "C"
