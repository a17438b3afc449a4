// All-gather of small per-rank records over peer memory, fused with the log-sum-exp merge that consumes them.
//
// Long-context decode splits the keys of one sequence over the GPUs; each rank ends its step with one record
// {m, l, O[D]} per query head (33 KB for 64 heads), and every rank needs all of them to merge.  Instead of a library
// all-gather between two kernels, rank r stores its records straight into slot r of every rank's gather buffer
// (plain 16-byte stores through NVLink peer mappings), publishes an epoch number with a system-scope release, and the
// merge kernel of each rank waits, with a bound, until every slot carries the current epoch.
//   buffers of one rank:  slots [2 parities][world][slot_floats]   flags [2 parities][world] (uint64 epoch)
// Epoch e uses parity e & 1: a rank can only push epoch e + 2 after it has seen every peer's flag e + 1, and a peer
// publishes e + 1 after it has finished reading epoch e, so two parities are enough.
// Nothing here waits without a limit: when a peer never publishes, the merge kernel records a time-out and returns.
#pragma once
#include <cuda_runtime.h>

#include "ptx_sm100.cuh"

namespace fusor {

constexpr int PX_MAX_WORLD = 16;

struct PeerPushParams {
    const float4* src;              // this rank's records, n_vec float4
    long long n_vec;
    uint8_t* base[PX_MAX_WORLD];    // every rank's exchange allocation as mapped on this GPU (own entry included)
    size_t flags_off;               // byte offset of the flags inside an allocation
    size_t slot_floats;             // capacity of one slot
    int world, rank;
    unsigned long long* epoch;      // local device counter: number of completed pushes; this push publishes *epoch + 1
    unsigned int* done;             // local, [world + 1], zero between launches
};

// The epoch lives in device memory, not in the launch parameters, so that a captured CUDA graph can be replayed: every
// rank launches the same sequence, so the counters agree.
// grid.y = destination rank; grid.x blocks copy the records; the last block to finish for a destination publishes
// the epoch there.  Stores to a peer are ordered before the flag by the system-scope fence + release store.
__global__ void peer_push_kernel(const PeerPushParams P) {
    const int dst_rank = blockIdx.y;
    const unsigned long long e = *reinterpret_cast<volatile unsigned long long*>(P.epoch) + 1;
    const size_t par = (size_t)(e & 1);
    float4* dst = reinterpret_cast<float4*>(P.base[dst_rank] + ((par * P.world + P.rank) * P.slot_floats) * 4);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < P.n_vec; i += (long long)gridDim.x * blockDim.x)
        dst[i] = P.src[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (atomicAdd(P.done + dst_rank, 1u) == gridDim.x - 1) {
            P.done[dst_rank] = 0;
            unsigned long long* flag = reinterpret_cast<unsigned long long*>(P.base[dst_rank] + P.flags_off) + par * P.world + P.rank;
            __threadfence_system();
            asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(flag), "l"(e) : "memory");
            if (atomicAdd(P.done + P.world, 1u) == (unsigned)P.world - 1) {  // every destination has been served
                P.done[P.world] = 0;
                *reinterpret_cast<volatile unsigned long long*>(P.epoch) = e;
                __threadfence();
            }
        }
    }
}

struct PeerMergeParams {
    const float* slots;                 // local: [2 parities][world][slot_floats]; a slot holds [n_rows][D + 2] records
    const unsigned long long* flags;    // local: [2 parities][world]
    const unsigned long long* epoch;    // local counter, already advanced by this step's push (same stream)
    size_t slot_floats;
    int world, D;
    long long n_rows;
    float* out;                         // [n_rows][D]
    int* err;
    long long wait_limit_cycles;
};

// One block per row.  Thread 0 waits (bounded) for every rank's epoch, then the block merges that row's records:
// M = max m, L = sum l e^(m - M), out = sum O e^(m - M) / L; a record with l == 0 contributes nothing.  The records were
// written by other GPUs: they are read with L2-only loads after the acquire, never from a stale L1 line.
__global__ void peer_merge_kernel(const PeerMergeParams P) {
    __shared__ int ready;
    const unsigned long long e = *P.epoch;
    const size_t par = (size_t)(e & 1);
    if (threadIdx.x == 0) {
        int ok = 1;
        const long long t0 = clock64();
        for (int r = 0; r < P.world && ok; ++r) {
            while (true) {
                unsigned long long v;
                asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(P.flags + par * P.world + r) : "memory");
                if (v >= e) break;
                if (clock64() - t0 > P.wait_limit_cycles) {
                    atomicCAS(P.err, 0, kErrWaitTimeout | (70 << 8));
                    ok = 0;
                    break;
                }
            }
        }
        ready = ok;
    }
    __syncthreads();
    if (!ready) return;
    const long long row = blockIdx.x;
    const long long rec = P.D + 2;
    const float* base = P.slots + par * P.world * P.slot_floats + row * rec;
    float M = -INFINITY;
    for (int p = 0; p < P.world; ++p) {
        const float* pr = base + (size_t)p * P.slot_floats;
        if (__ldcg(pr + 1) != 0.0f) M = fmaxf(M, __ldcg(pr));
    }
    float L = 0.0f;
    for (int p = 0; p < P.world; ++p) {
        const float* pr = base + (size_t)p * P.slot_floats;
        if (__ldcg(pr + 1) != 0.0f) L += __ldcg(pr + 1) * __expf(__ldcg(pr) - M);
    }
    for (int d = threadIdx.x; d < P.D; d += blockDim.x) {
        float acc = 0.0f;
        for (int p = 0; p < P.world; ++p) {
            const float* pr = base + (size_t)p * P.slot_floats;
            if (__ldcg(pr + 1) != 0.0f) acc += __ldcg(pr + 2 + d) * __expf(__ldcg(pr) - M);
        }
        P.out[row * P.D + d] = acc / L;
    }
}

}  // namespace fusor
