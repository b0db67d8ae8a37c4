// CPU model of the cross-rank protocols the fused kernels rely on, with ranks as threads and C++ atomics in
// place of st.release.sys / ld.acquire.sys. It checks, under randomised scheduling, the claims the GPU code
// is built on:
//
//   1. epoch flags + two buffer halves (AG-GEMM workspace, all-to-all receive buffers, LL gather buffers):
//      a rank starts call e+1 right after finishing call e, with no barrier; a consumer of call e never
//      sees data of another call in the half it reads, because a peer can only write call e+2 into that half
//      after this rank has pushed call e+1, which it does after it finished reading call e.
//   2. a flag that never comes (a dead peer) makes the waiter give up after its limit and report
//      {peer, expected, seen} instead of spinning forever; later waits return at once (sticky abort).
//   3. the top-bit-flip grid barrier works across launches with different numbers of participants.
//   4. LL packets (payload and flag in one 16-byte store, the receiver waits for flag == call number) with two
//      buffer halves and no barrier: the exchange of the sequence-parallel decode and of the LL all-gather. Here a
//      writer that ran two calls ahead would make the reader wait forever for a flag value that was overwritten,
//      so the model also proves that no rank can get two calls ahead.
//   5. claim / copy / arrive with the last arriver publishing (the in-launch row staging of the grouped GEMM and the
//      sliced pushers of the AG-GEMM): a consumer that sees a block's flag sees every row of it, and the cursor and the
//      arrival counters are back at zero when the call ends.
//
// Build and run: g++ -O2 -std=c++17 -pthread flag_protocol_model.cc -o model && ./model [ranks] [calls] [seed]
// Prints "OK ..." and exits 0, or the first violation and exits 1.
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <thread>
#include <vector>

namespace {

constexpr int kBlocks = 4;      // 128-row blocks per rank segment
constexpr int kWords = 64;      // payload words per block

struct Status {
    std::atomic<int> abort{0};
    std::atomic<int> code{0};
    int peer = -1;
    uint64_t expected = 0, seen = 0;
};

struct Rank {
    // workspace[half][src][block][word], flags[half][src][block]
    std::vector<std::atomic<uint64_t>> ws;
    std::vector<std::atomic<uint32_t>> flags;
    Status status;
    explicit Rank(int world) : ws(2ull * world * kBlocks * kWords), flags(2ull * world * kBlocks) {
        for (auto& w : ws) w.store(~0ull, std::memory_order_relaxed);
        for (auto& f : flags) f.store(0, std::memory_order_relaxed);
    }
};

inline uint64_t pattern(int src, uint32_t call, int block, int word) {
    return (static_cast<uint64_t>(src) << 48) | (static_cast<uint64_t>(call) << 16) | (static_cast<uint64_t>(block) << 8) | static_cast<uint64_t>(word);
}

// bounded acquire wait, the CPU twin of wait_flag_ge_sys
bool wait_flag_ge(std::atomic<uint32_t>& flag, uint32_t epoch, Status& st, int peer, std::chrono::milliseconds limit) {
    const auto t0 = std::chrono::steady_clock::now();
    uint32_t spins = 0;
    while (true) {
        const uint32_t v = flag.load(std::memory_order_acquire);
        if (static_cast<int32_t>(v - epoch) >= 0) return true;
        if ((++spins & 255u) == 0) {
            if (st.abort.load(std::memory_order_relaxed)) return false;
            if (std::chrono::steady_clock::now() - t0 > limit) {
                int expected_code = 0;
                if (st.code.compare_exchange_strong(expected_code, 1)) {
                    st.peer = peer;
                    st.expected = epoch;
                    st.seen = v;
                }
                st.abort.store(1, std::memory_order_release);
                return false;
            }
            std::this_thread::yield();
        }
    }
}

std::atomic<int> g_violations{0};

void run_rank(int rank, int world, int calls, unsigned seed, std::vector<Rank*>& ranks, int dead_rank, int dead_call,
              std::chrono::milliseconds limit) {
    std::mt19937 rng(seed * 7919u + rank);
    auto jitter = [&]() {
        const unsigned r = rng() % 16;
        if (r == 0) std::this_thread::sleep_for(std::chrono::microseconds(rng() % 200));
        else if (r < 4) std::this_thread::yield();
    };
    Rank& me = *ranks[rank];
    for (uint32_t e = 1; e <= static_cast<uint32_t>(calls); ++e) {
        const int half = e & 1;
        if (rank == dead_rank && static_cast<int>(e) >= dead_call) return;  // a peer that stops notifying
        // ---- "pusher": write this rank's blocks into every peer's half, then release the block's flag
        for (int hop = 1; hop < world; ++hop) {
            const int dst = (rank - hop + world) % world;
            Rank& peer = *ranks[dst];
            for (int b = 0; b < kBlocks; ++b) {
                jitter();
                const size_t base = ((static_cast<size_t>(half) * world + rank) * kBlocks + b) * kWords;
                for (int w = 0; w < kWords; ++w) peer.ws[base + w].store(pattern(rank, e, b, w), std::memory_order_relaxed);
                peer.flags[(static_cast<size_t>(half) * world + rank) * kBlocks + b].store(e, std::memory_order_release);
            }
        }
        // ---- "consumer": segments in ring order from the own one, wait per block, then read and verify
        for (int s = 1; s < world; ++s) {
            const int src = (rank + s) % world;
            for (int b = 0; b < kBlocks; ++b) {
                jitter();
                auto& flag = me.flags[(static_cast<size_t>(half) * world + src) * kBlocks + b];
                if (!wait_flag_ge(flag, e, me.status, src, limit)) return;  // reported; drain without touching peers
                const size_t base = ((static_cast<size_t>(half) * world + src) * kBlocks + b) * kWords;
                for (int w = 0; w < kWords; ++w) {
                    const uint64_t v = me.ws[base + w].load(std::memory_order_relaxed);
                    if (v != pattern(src, e, b, w)) {
                        if (g_violations.fetch_add(1) == 0)
                            std::fprintf(stderr, "VIOLATION rank %d call %u: block %d of rank %d word %d holds %llx, wanted %llx\n", rank, e, b,
                                         src, w, static_cast<unsigned long long>(v), static_cast<unsigned long long>(pattern(src, e, b, w)));
                        return;
                    }
                }
            }
        }
    }
}

// top-bit-flip barrier: participant 0 adds 0x80000000 - (n - 1), the others add 1; everyone waits for the top
// bit to differ from what its own add saw
bool grid_barrier_model(unsigned seed) {
    std::atomic<uint32_t> counter{0};
    std::mt19937 rng(seed);
    for (int round = 0; round < 200; ++round) {
        const int n = 1 + static_cast<int>(rng() % 12);
        std::atomic<int> arrived{0}, passed_early{0};
        std::vector<std::thread> th;
        for (int i = 0; i < n; ++i)
            th.emplace_back([&, i]() {
                if (i % 3 == 1) std::this_thread::yield();
                arrived.fetch_add(1);
                const uint32_t old = counter.fetch_add(i == 0 ? 0x80000000u - static_cast<uint32_t>(n - 1) : 1u, std::memory_order_acq_rel);
                while (((old ^ counter.load(std::memory_order_acquire)) & 0x80000000u) == 0) std::this_thread::yield();
                if (arrived.load() != n) passed_early.fetch_add(1);
            });
        for (auto& t : th) t.join();
        if (passed_early.load() != 0 || (counter.load() & 0x7fffffffu) != 0) {
            std::fprintf(stderr, "VIOLATION grid barrier: round %d with %d participants, counter %x\n", round, n, counter.load());
            return false;
        }
    }
    return true;
}

// ---- LL packets: one 128-bit word per (half, source), modelled as payload << 32 | flag in a 64-bit atomic
struct LLRank {
    std::vector<std::atomic<uint64_t>> slot;   // [2][world]
    std::atomic<int> error{0};
    explicit LLRank(int world) : slot(2ull * world) {
        for (auto& s : slot) s.store(0, std::memory_order_relaxed);
    }
};

void run_ll_rank(int rank, int world, int calls, unsigned seed, std::vector<LLRank*>& ranks, std::chrono::milliseconds limit) {
    std::mt19937 rng(seed * 104729u + rank);
    for (uint32_t e = 1; e <= static_cast<uint32_t>(calls); ++e) {
        const int half = e & 1;
        if (rng() % 8 == 0) std::this_thread::yield();
        if (rng() % 64 == 0) std::this_thread::sleep_for(std::chrono::microseconds(rng() % 300));
        for (int p = 0; p < world; ++p)  // every rank, itself included, gets (payload = rank * 1000003 + e, flag = e)
            ranks[p]->slot[static_cast<size_t>(half) * world + rank].store(
                (static_cast<uint64_t>(static_cast<uint32_t>(rank * 1000003 + e)) << 32) | e, std::memory_order_release);
        for (int src = 0; src < world; ++src) {
            const auto t0 = std::chrono::steady_clock::now();
            uint32_t spins = 0;
            while (true) {
                const uint64_t v = ranks[rank]->slot[static_cast<size_t>(half) * world + src].load(std::memory_order_acquire);
                if (static_cast<uint32_t>(v) == e) {
                    if (static_cast<uint32_t>(v >> 32) != static_cast<uint32_t>(src * 1000003 + e)) ranks[rank]->error.store(2);
                    break;
                }
                if ((++spins & 1023u) == 0) {
                    if (std::chrono::steady_clock::now() - t0 > limit) {
                        ranks[rank]->error.store(1);   // the flag it waits for was skipped or overwritten
                        return;
                    }
                    std::this_thread::yield();
                }
            }
        }
    }
}

// ---- claim, copy, arrive; the last arriver publishes (row staging of the grouped GEMM, sliced AG pushers)
// Workers (the epilogue warps of all CTAs / the pusher CTAs) claim groups of a block from one cursor, write the group's
// rows with plain stores, then add to the block's arrival counter (acq_rel). The worker whose add completes the block
// resets the counter for the next call and release-stores the block's flag = call number. Consumers (the TMA producers
// / the peer's MMA side) acquire-wait for flag >= call and must then see this call's value in EVERY row of the block.
// The cursor is rewound by the last worker to leave the call (an exit counter), as the kernel does.
bool staging_model(unsigned seed, int calls) {
    constexpr int kBlocks = 12, kGroups = 4, kRows = 3, kWorkers = 6, kConsumers = 3;
    std::vector<std::atomic<uint32_t>> rows(kBlocks * kGroups * kRows), flag(kBlocks), arrive(kBlocks);
    for (auto& r : rows) r.store(0, std::memory_order_relaxed);
    for (auto& f : flag) f.store(0, std::memory_order_relaxed);
    for (auto& a : arrive) a.store(0, std::memory_order_relaxed);
    std::atomic<uint32_t> cursor{0}, exits{0}, start{0};
    std::atomic<int> bad{0};
    auto worker = [&](int id) {
        std::mt19937 rng(seed * 7919u + id);
        for (uint32_t e = 1; e <= static_cast<uint32_t>(calls); ++e) {
            while (start.load(std::memory_order_acquire) < e) std::this_thread::yield();   // the launch of call e
            while (true) {
                const uint32_t item = cursor.fetch_add(1, std::memory_order_relaxed);
                if (item >= kBlocks * kGroups) break;
                const int b = item / kGroups, g = item % kGroups;
                if (rng() % 4 == 0) std::this_thread::yield();
                for (int r = 0; r < kRows; ++r) rows[(b * kGroups + g) * kRows + r].store(e * 1000u + b, std::memory_order_relaxed);
                if (arrive[b].fetch_add(1, std::memory_order_acq_rel) == kGroups - 1) {
                    arrive[b].store(0, std::memory_order_relaxed);
                    flag[b].store(e, std::memory_order_release);
                }
            }
            if (exits.fetch_add(1, std::memory_order_acq_rel) == kWorkers + kConsumers - 1) {
                cursor.store(0, std::memory_order_relaxed);
                exits.store(0, std::memory_order_relaxed);
                start.store(e + 1, std::memory_order_release);   // the next launch starts after this one has ended
            }
        }
    };
    auto consumer = [&](int id) {
        for (uint32_t e = 1; e <= static_cast<uint32_t>(calls); ++e) {
            while (start.load(std::memory_order_acquire) < e) std::this_thread::yield();
            for (int b = id; b < kBlocks; b += kConsumers) {
                uint32_t spins = 0;
                while (static_cast<int32_t>(flag[b].load(std::memory_order_acquire) - e) < 0)
                    if ((++spins & 255u) == 0) std::this_thread::yield();
                for (int i = 0; i < kGroups * kRows; ++i)
                    if (rows[b * kGroups * kRows + i].load(std::memory_order_relaxed) != e * 1000u + b) bad.store(1);
            }
            if (exits.fetch_add(1, std::memory_order_acq_rel) == kWorkers + kConsumers - 1) {
                cursor.store(0, std::memory_order_relaxed);
                exits.store(0, std::memory_order_relaxed);
                start.store(e + 1, std::memory_order_release);
            }
        }
    };
    start.store(1, std::memory_order_release);
    std::vector<std::thread> th;
    for (int i = 0; i < kWorkers; ++i) th.emplace_back(worker, i);
    for (int i = 0; i < kConsumers; ++i) th.emplace_back(consumer, i);
    for (auto& t : th) t.join();
    bool ok = bad.load() == 0 && cursor.load() == 0;
    for (auto& a : arrive) ok = ok && a.load() == 0;
    if (!ok) std::fprintf(stderr, "VIOLATION staging: a consumer saw a row of another call, or a counter was left non-zero\n");
    return ok;
}

}  // namespace

int main(int argc, char** argv) {
    const int world = argc > 1 ? std::atoi(argv[1]) : 4;
    const int calls = argc > 2 ? std::atoi(argv[2]) : 200;
    const unsigned seed = argc > 3 ? static_cast<unsigned>(std::atoi(argv[3])) : 1u;
    // 1. healthy run
    {
        std::vector<Rank*> ranks;
        for (int r = 0; r < world; ++r) ranks.push_back(new Rank(world));
        std::vector<std::thread> th;
        for (int r = 0; r < world; ++r) th.emplace_back(run_rank, r, world, calls, seed, std::ref(ranks), -1, 0, std::chrono::milliseconds(20000));
        for (auto& t : th) t.join();
        bool bad = g_violations.load() != 0;
        for (auto* r : ranks) {
            bad = bad || r->status.code.load() != 0;
            delete r;
        }
        if (bad) {
            std::fprintf(stderr, "healthy run failed\n");
            return 1;
        }
    }
    // 2. a peer that stops notifying: every other rank gives up within the limit and says who was missing
    {
        const int dead = world - 1, dead_call = calls / 2 + 1;
        std::vector<Rank*> ranks;
        for (int r = 0; r < world; ++r) ranks.push_back(new Rank(world));
        std::vector<std::thread> th;
        const auto t0 = std::chrono::steady_clock::now();
        for (int r = 0; r < world; ++r) th.emplace_back(run_rank, r, world, calls, seed + 1, std::ref(ranks), dead, dead_call, std::chrono::milliseconds(150));
        for (auto& t : th) t.join();
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        bool ok = g_violations.load() == 0;
        int reported = 0;
        for (int r = 0; r < world; ++r) {
            if (r != dead && ranks[r]->status.code.load() == 1) {
                ++reported;
                ok = ok && ranks[r]->status.abort.load() == 1 && ranks[r]->status.expected >= static_cast<uint64_t>(dead_call) - 0;
            }
        }
        // the ranks that depend on the dead one directly report it; the others report the rank they starved on
        ok = ok && reported == world - 1 && ms < 20000;
        for (auto* r : ranks) delete r;
        if (!ok) {
            std::fprintf(stderr, "dead-peer run failed: %d of %d ranks reported, %lld ms\n", reported, world - 1, static_cast<long long>(ms));
            return 1;
        }
    }
    // 3. grid barrier with changing participant counts
    if (!grid_barrier_model(seed)) return 1;
    // 4. LL exchange with equality flags, two halves, no barrier
    {
        std::vector<LLRank*> ranks;
        for (int r = 0; r < world; ++r) ranks.push_back(new LLRank(world));
        std::vector<std::thread> th;
        for (int r = 0; r < world; ++r) th.emplace_back(run_ll_rank, r, world, calls * 4, seed + 2, std::ref(ranks), std::chrono::milliseconds(20000));
        for (auto& t : th) t.join();
        int bad = 0;
        for (auto* r : ranks) {
            bad |= r->error.load();
            delete r;
        }
        if (bad) {
            std::fprintf(stderr, "LL exchange failed (%s)\n", bad == 1 ? "a flag value was skipped or overwritten" : "payload of another call");
            return 1;
        }
    }
    // 5. claim / copy / arrive, last arriver publishes; counters return to zero for the next call
    if (!staging_model(seed + 3, calls)) return 1;
    std::printf("OK world=%d calls=%d seed=%u\n", world, calls, seed);
    return 0;
}
