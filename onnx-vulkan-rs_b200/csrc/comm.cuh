// Flags that the GPUs of one box exchange through each other's memory.
//
// Every rank owns one OvkCommFlags block in its own device memory and knows the
// address of every other rank's block (a peer mapping).  A rank announces
// something by STORING the current call number (the epoch) into its slot of
// every peer's block; a rank waits by POLLING its own block, so polls never
// cross NVLink.  Two announcements per collective call:
//   ready[r] = e   rank r's stream has reached call e: everything it enqueued
//                  before - in particular the readers of the buffers the peers
//                  are about to overwrite - has finished
//   done[r]  = e   every store of rank r's call e into this rank's memory has
//                  been issued and made visible (fence, then the flag)
// Epochs only grow, so a waiter compares with >= (as a signed difference) and a
// rank that is one call ahead never confuses a slower one.  Every wait is
// bounded by a clock limit; when it runs out the caller records
// OVK_DEV_TIMEOUT_PEER in the context's status word and carries on without
// waiting, so a missing peer ends in OVK_TIMEOUT from ovk_flush, not in a hang.
#pragma once

#include <cstdint>

constexpr int OVK_MAX_RANKS = 8;

struct OvkCommFlags {
    uint32_t ready[16];
    uint32_t done[16];
    uint32_t cta_done;  // CTAs of the local kernel that have finished their stores (reset by the last one)
    uint32_t pad[31];
};
static_assert(sizeof(OvkCommFlags) == 256, "one flag block is 256 bytes");

// What a kernel that stores into peers' memory needs to know.
struct OvkCommView {
    OvkCommFlags *flags[OVK_MAX_RANKS];  // flags[rank] is this GPU's own block
    int rank, world;
    uint32_t epoch;
    long long wait_cycles;
};

#ifdef __CUDACC__
namespace comm {

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// the same, for a word only blocks of this GPU write
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One 16-byte store to the same offset of EVERY rank's buffer: the address is a multicast mapping of the
// ranks' buffers, the store crosses this GPU's links once and the NVSwitch delivers it to all of them
// (this GPU's own copy included).
__device__ __forceinline__ void st_multicast16(void *mc_addr, uint4 v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
                 "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                 : "memory");
}

// Called by one whole warp: lane d stores the epoch into slot `rank` of peer d's array.
__device__ __forceinline__ void announce(const OvkCommView &c, bool done_flag, int lane)
{
    if (lane < c.world) {
        OvkCommFlags *f = c.flags[lane];
        st_release_sys(done_flag ? &f->done[c.rank] : &f->ready[c.rank], c.epoch);
    }
}

// Called by one whole warp: lane s polls slot s of this GPU's own array until every
// rank's epoch has arrived.  Returns false when the clock limit ran out first.
__device__ __forceinline__ bool wait_all(const OvkCommView &c, bool done_flag, int lane)
{
    const OvkCommFlags *own = c.flags[c.rank];
    const uint32_t *slot = done_flag ? &own->done[lane & 15] : &own->ready[lane & 15];
    const bool mine = lane < c.world && lane != c.rank;
    const long long t0 = clock64();
    for (;;) {
        const bool here = !mine || int32_t(ld_acquire_sys(slot) - c.epoch) >= 0;
        if (__all_sync(0xffffffffu, here))
            return true;
        if (__any_sync(0xffffffffu, clock64() - t0 > c.wait_cycles))
            return false;
        __nanosleep(200);
    }
}

}  // namespace comm
#endif
