// All-gather of small per-rank records over peer memory, fused with the log-sum-exp merge that consumes them.
//
// Long-context decode splits the keys of one sequence over the GPUs; each rank ends its step with one record
// {m, l, O[D]} per query head (33 KB for 64 heads), and every rank needs all of them to merge.  Instead of a library
// all-gather between two kernels, rank r stores its records straight into slot r of every rank's gather buffer
// (plain 16-byte stores through NVLink peer mappings), publishes an epoch number with a system-scope release, and the
// merge of each rank waits, with a bound, until every slot carries the current epoch.
//   buffers of one rank:  slots [2 parities][world][slot_floats]   flags [2 parities][world] (uint64 epoch)
// Epoch e uses parity e & 1: a rank can only push epoch e + 2 after it has seen every peer's flag e + 1, and a peer
// publishes e + 1 after it has finished reading epoch e, so two parities are enough.
// Two producers of the records exist: decode_combine_exchange_kernel (decode_splitkv.cuh), which merges a rank's split-KV
// records per query head, stores the result on every rank, publishes, waits and merges over the ranks in one launch, and
// peer_push_merge_kernel, which does the same for records the caller already holds.  Peer memory is only ever written by
// these kernels, never read.
// Nothing here waits without a limit: when a peer never publishes, the merge records a time-out and returns.
#pragma once
#include <cuda_runtime.h>

#include "ptx_sm100.cuh"

namespace fusor {

constexpr int PX_MAX_WORLD = 16;

// Where a rank's records go: every rank's exchange allocation as mapped on this GPU (own entry included).
struct PeerTargets {
    uint8_t* base[PX_MAX_WORLD];
    size_t flags_off;               // byte offset of the flags inside an allocation
    size_t slot_floats;             // capacity of one slot
    int world, rank;
    // The epoch lives in device memory, not in the launch parameters, so that a captured CUDA graph can be replayed:
    // every rank launches the same sequence, so the counters agree.  A step publishes *epoch + 1; the merge that ends
    // the step advances the counter.
    unsigned long long* epoch;
    unsigned int* done;             // local, [4] block counters, zero between launches
};

__device__ __forceinline__ float* peer_slot(const PeerTargets& T, int dst_rank, unsigned long long e) {
    return reinterpret_cast<float*>(T.base[dst_rank] + (((size_t)(e & 1) * T.world + T.rank) * T.slot_floats) * 4);
}

// Called by one thread after this rank's stores to every peer have been fenced at system scope and the CTA's other
// threads have passed a barrier: tells every rank that slot `rank` of parity e & 1 holds epoch e.
__device__ __forceinline__ void peer_publish(const PeerTargets& T, unsigned long long e) {
    __threadfence_system();
    for (int r = 0; r < T.world; ++r) {
        unsigned long long* flag = reinterpret_cast<unsigned long long*>(T.base[r] + T.flags_off) + (size_t)(e & 1) * T.world + T.rank;
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(flag), "l"(e) : "memory");
    }
}

struct PeerMergeParams {
    const float* slots;                 // local: [2 parities][world][slot_floats]; a slot holds [n_rows][D + 2] records
    const unsigned long long* flags;    // local: [2 parities][world]
    unsigned long long* epoch;          // local counter; this step is epoch *epoch + 1
    unsigned int* done;                 // local block counter (index 2 of the exchange's counters), zero between launches
    size_t slot_floats;
    int world, D;
    long long n_rows;
    float* out;                         // [n_rows][D]
    int* err;
    long long wait_limit_cycles;
};

// Threads 0 .. world-1 of a block each wait (bounded) for one rank's epoch; returns whether all arrived.  A block that
// finds a time-out already recorded gives up after one look, so a lost peer costs one wait limit, not one per wave.
__device__ __forceinline__ bool peer_wait_all(const unsigned long long* flags, int world, unsigned long long e, int* err,
                                              long long limit) {
    int ok = 1;
    if ((int)threadIdx.x < world) {
        const unsigned long long* f = flags + (size_t)(e & 1) * world + threadIdx.x;
        const long long t0 = clock64();
        while (true) {
            unsigned long long v;
            asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(f) : "memory");
            if (v >= e) break;
            if (*reinterpret_cast<volatile int*>(err) != 0) { ok = 0; break; }
            if (clock64() - t0 > limit) {
                atomicCAS(err, 0, kErrWaitTimeout | (70 << 8));
                ok = 0;
                break;
            }
        }
    }
    return __syncthreads_and(ok) != 0;
}

// Merge of one row's records over the ranks: M = max m, L = sum l e^(m - M), out = sum O e^(m - M) / L; a record with
// l == 0 contributes nothing, and a row whose records are all empty gives zeros (the same rule as lse_combine_kernel).
// The records were written by other GPUs: they are read with L2-only loads after the acquire, never from a stale L1 line.
__device__ __forceinline__ void peer_merge_row(const float* slots, size_t slot_floats, int world, unsigned long long e, long long row,
                                               int D, float* out) {
    const long long rec = D + 2;
    const float* base = slots + (size_t)(e & 1) * world * slot_floats + row * rec;
    float M = -INFINITY;
    for (int p = 0; p < world; ++p) {
        const float* pr = base + (size_t)p * slot_floats;
        if (__ldcg(pr + 1) != 0.0f) M = fmaxf(M, __ldcg(pr));
    }
    float L = 0.0f;
    for (int p = 0; p < world; ++p) {
        const float* pr = base + (size_t)p * slot_floats;
        if (__ldcg(pr + 1) != 0.0f) L += __ldcg(pr + 1) * __expf(__ldcg(pr) - M);
    }
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.0f;
        for (int p = 0; p < world; ++p) {
            const float* pr = base + (size_t)p * slot_floats;
            if (__ldcg(pr + 1) != 0.0f) acc += __ldcg(pr + 2 + d) * __expf(__ldcg(pr) - M);
        }
        out[row * D + d] = acc * inv;
    }
}

// Ends a step: the last block to finish advances the epoch counter.
__device__ __forceinline__ void peer_step_done(unsigned long long* epoch, unsigned int* done, unsigned long long e) {
    __syncthreads();
    if (threadIdx.x == 0) {
        if (atomicAdd(done, 1u) == gridDim.x - 1) {
            *done = 0;
            *reinterpret_cast<volatile unsigned long long*>(epoch) = e;
            __threadfence();
        }
    }
}

struct PeerPushMergeParams {
    const float4* src;   // this rank's records, n_vec float4
    long long n_vec;
    PeerTargets T;
    PeerMergeParams M;
};

// Push, publish, wait and merge in one launch, for records the caller already holds.  The grid is at most one block per
// SM, so every block is resident: a block only waits for the peers after all of this rank's blocks have stored their
// share (the last one to finish publishes), and no block waits on a block that has not started.
__global__ void peer_push_merge_kernel(const PeerPushMergeParams P) {
    const unsigned long long e = *reinterpret_cast<volatile unsigned long long*>(P.T.epoch) + 1;
    for (int r = 0; r < P.T.world; ++r) {
        float4* dst = reinterpret_cast<float4*>(peer_slot(P.T, r, e));
        for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < P.n_vec; i += (long long)gridDim.x * blockDim.x)
            dst[i] = P.src[i];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(P.T.done, 1u) == gridDim.x - 1) {
        *P.T.done = 0;
        peer_publish(P.T, e);
    }
    if (peer_wait_all(P.M.flags, P.M.world, e, P.M.err, P.M.wait_limit_cycles))
        for (long long row = blockIdx.x; row < P.M.n_rows; row += gridDim.x)
            peer_merge_row(P.M.slots, P.M.slot_floats, P.M.world, e, row, P.M.D, P.M.out);
    peer_step_done(P.M.epoch, P.M.done, e);
}

}  // namespace fusor
