// Host-side helpers shared by the translation units that launch the kernels:
// how a dense column of height k is spread over a worker, the chunk length, and
// the process-wide launch counter.
#pragma once
#include <atomic>
#include <cstdint>
#include <cstdlib>

#include "common.cuh"

namespace bidmat {

// Kernels launched by this library in this process (all devices).
inline std::atomic<long long> g_launches{0};

// How a dense column of height k is spread over a worker.
struct Shape {
    int vec;   // 16-byte vectors (4 floats / 2 doubles) when k allows and the pointers are aligned, else 1
    int lpv;   // lanes per worker
    int nt;    // VEC-wide elements per lane
    int tiles; // k-tiles of width lpv*nt*vec
};

inline Shape pick_shape(int k, bool aligned16, int wide = 4) {
    Shape s;
    s.vec = (aligned16 && (k % wide == 0)) ? wide : 1;
    const int kv = k / s.vec;
    if (kv <= 8) { s.lpv = 8; s.nt = 1; }
    else if (kv <= 16) { s.lpv = 16; s.nt = 1; }
    else if (kv <= 32) { s.lpv = 32; s.nt = 1; }
    else if (kv <= 64) { s.lpv = 32; s.nt = 2; }
    else { s.lpv = 32; s.nt = 4; }
    const int tile = s.lpv * s.nt * s.vec;
    s.tiles = (k + tile - 1) / tile;
    return s;
}

inline bool is16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int env_int(const char *name, int dflt) {
    const char *v = getenv(name);
    if (!v || !*v) return dflt;
    return atoi(v);
}

// Chunk length: about kTargetChunks chunks per launch (8 per resident worker
// slot of a 148-SM part), never fewer than 64 nor more than 4096 nonzeros per
// chunk.  BIDMAT_B200_CHUNK overrides (tests use tiny chunks to force runs
// across chunk boundaries).
constexpr long long kTargetChunks = 148LL * 16 * 8;

inline int pick_chunk(long long nnz, int lpv) {
    int forced = env_int("BIDMAT_B200_CHUNK", 0);
    long long c;
    if (forced > 0) c = forced;
    else {
        const long long target = env_int("BIDMAT_B200_TARGET_CHUNKS", (int)kTargetChunks);
        c = (nnz + target - 1) / target;
        if (c < 64) c = 64;
        if (c > 4096) c = 4096;
    }
    c = ((c + lpv - 1) / lpv) * lpv;
    return (int)c;
}

// Upper bound on the number of chunks pick_chunk can give to the whole list of
// nnz nonzeros or to any slice of it.
inline long long max_chunks_for(long long nnz, int lpv) {
    const int chunk_all = pick_chunk(nnz, lpv);
    long long cap = (nnz + chunk_all - 1) / chunk_all;
    long long by64 = (nnz + 63) / 64 + 1;
    const long long target = env_int("BIDMAT_B200_TARGET_CHUNKS", (int)kTargetChunks);
    long long alt = by64 < target + 1 ? by64 : target + 1;
    return alt > cap ? alt : cap;
}

// Expects `kWideVec` (4 for float, 2 for double) as a constant in the calling scope.
#define DISPATCH_SHAPE(S, CALL)                                                     \
    do {                                                                            \
        if ((S).vec > 1) {                                                          \
            if ((S).lpv == 8) { CALL(kWideVec, 8, 1); }                             \
            else if ((S).lpv == 16) { CALL(kWideVec, 16, 1); }                      \
            else if ((S).nt == 1) { CALL(kWideVec, 32, 1); }                        \
            else if ((S).nt == 2) { CALL(kWideVec, 32, 2); }                        \
            else { CALL(kWideVec, 32, 4); }                                         \
        } else {                                                                    \
            if ((S).lpv == 8) { CALL(1, 8, 1); }                                    \
            else if ((S).lpv == 16) { CALL(1, 16, 1); }                             \
            else if ((S).nt == 1) { CALL(1, 32, 1); }                               \
            else if ((S).nt == 2) { CALL(1, 32, 2); }                               \
            else { CALL(1, 32, 4); }                                                \
        }                                                                           \
    } while (0)

inline unsigned blocks_for(long long workers, int lpv) {
    long long threads = workers * lpv;
    return (unsigned)((threads + kThreads - 1) / kThreads);
}


inline size_t ga_part_floats(int k, long long nnz, int chunk) {
    const long long nchunks = (nnz + chunk - 1) / chunk;
    return (size_t)nchunks * 2 * (size_t)k;
}

}  // namespace bidmat
