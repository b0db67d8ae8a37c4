// "LL" (low-latency) packets: every 16-byte packet carries 8 bytes of payload and two copies of
// a 32-bit flag, so the receiver learns that the payload has arrived from the payload itself —
// no separate signal, no fence on the sender. Doubles the bytes on the wire; wins for messages
// of a few KB where one NVLink round trip dominates.
// (reference kernels/nvidia/low_latency_allgather.py:531-567 `_pack_ll_block` / `_recv_ll_block`.)
#pragma once
#include "signal.cuh"

namespace tdist {

__device__ __forceinline__ void ll_store(void* packet, uint64_t payload, uint32_t flag) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(packet),
                 "r"(static_cast<uint32_t>(payload)), "r"(flag), "r"(static_cast<uint32_t>(payload >> 32)), "r"(flag)
                 : "memory");
}

// The same packet through an NVSwitch multicast address: the switch replicates the store to every device bound to
// the multicast object (reference low_latency_allgather.py:570-697 `_recv_ll_and_multimem_st*`, multimem.st.b64).
__device__ __forceinline__ void ll_store_multimem(void* mc_packet, uint64_t payload, uint32_t flag) {
    asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_packet),
                 "r"(static_cast<uint32_t>(payload)), "r"(flag), "r"(static_cast<uint32_t>(payload >> 32)), "r"(flag)
                 : "memory");
}

// Spins until both flag copies of the packet equal `flag`; bounded like every other wait.
__device__ __forceinline__ bool ll_load(const void* packet, uint32_t flag, uint64_t* payload, const WaitCtx& w,
                                        int peer, int index) {
    uint32_t d0, f0, d1, f1;
    uint32_t spins = 0;
    uint64_t t0 = 0;
    const uint64_t limit = w.timeout_ns ? w.timeout_ns : kDefaultTimeoutNs;
    while (true) {
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(d0), "=r"(f0), "=r"(d1), "=r"(f1)
                     : "l"(packet)
                     : "memory");
        if (f0 == flag && f1 == flag) {
            *payload = static_cast<uint64_t>(d0) | (static_cast<uint64_t>(d1) << 32);
            return true;
        }
        if ((++spins & 127u) == 0) {
            if (aborted(w)) break;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit) {
                report_timeout(w, kStatusFlagTimeout, peer, index, flag, f0, 200);
                break;
            }
        }
    }
    *payload = 0;
    return false;
}

}  // namespace tdist
