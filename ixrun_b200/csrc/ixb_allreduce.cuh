// One-shot all-reduce (sum) of a short fp32 vector over peer memory, for the partial outputs of row-parallel
// packed linears (o_proj / down_proj shards): out_f values per token, 20 KB for the 27B hybrid.
//
// The reference is single-GPU; its tensor-parallel form needs one sum of out_f values per row-parallel layer.
// A library all-reduce costs a launch of its own plus its protocol (15 .. 20 us eagerly, and it could not be
// captured in a CUDA graph on this pool); at this size the transfer itself is a few hundred nanoseconds of
// NVLink time, so the whole exchange is done by one small kernel with plain peer stores and loads:
//
//   every rank owns one buffer that all ranks can address (peer pointers):
//     slots  [2 parities][W ranks][n_max] fp32      flags [W ranks][ctas] uint32      epoch [ctas] uint32
//   CTA c of rank r, call number e (epoch[c] + 1), parity e & 1:
//     1. stores its 1024 values of the local partial vector into slot (parity, r) of EVERY rank's buffer,
//     2. fences (system scope), then stores e into flags[r][c] of every rank's buffer,
//     3. waits until flags[s][c] >= e for every sender s in ITS OWN buffer -- a bounded wait: after
//        kArSpinLimit polls it records an error word and goes on (and later calls stop waiting after 64 polls) --
//     4. sums slots (parity, 0 .. W-1) of its own buffer in rank order (every rank gets the same bits), adds the
//        bias, writes y (bf16 or fp32), and stores e into epoch[c].
// Two parities are enough: a rank can only reach call e + 2 after every other rank has sent call e + 1, which each
// does after it has finished reading call e.  Nothing here is a multicast or a TMA load; NVLink carries plain
// stores (data, flags) only, all loads are local.  The kernel takes part in programmatic dependent launch like
// k_p6_mma (it waits for the kernel ahead of it before it reads the partial vector).
#pragma once
#include "ixb_common.cuh"

namespace ixb {

constexpr int kArMaxWorld = 8;
constexpr int kArThreads = 256;
constexpr int kArPerCta = kArThreads * 4;                 // fp32 values per CTA
constexpr uint32_t kArSpinLimit = 1u << 22;               // polls (>= 32 ns each) before a wait gives up

struct ArPeers {
    float *slots[kArMaxWorld];                            // every rank's slots, as seen from this rank
    uint32_t *flags[kArMaxWorld];                         // every rank's flags
};

__host__ __device__ __forceinline__ size_t ar_slots_bytes(int world, int64_t n_max) { return (size_t)2 * world * n_max * 4; }
__host__ __device__ __forceinline__ uint32_t ar_ctas(int64_t n_max) { return (uint32_t)((n_max + kArPerCta - 1) / kArPerCta); }

template <int W>
__global__ void __launch_bounds__(kArThreads)
k_allreduce_oneshot(ArPeers peers, const float *__restrict__ x, int rank, uint32_t n, uint32_t n_max,
                    const __nv_bfloat16 *__restrict__ bias, void *y, int y_f32, uint32_t *epoch, uint32_t *err)
{
    __shared__ uint32_t e_s;
    const uint32_t c = blockIdx.x, ctas = gridDim.x, tid = threadIdx.x;
    asm volatile("griddepcontrol.launch_dependents;");
    const uint32_t i = (c * kArThreads + tid) * 4u;
    const bool valid = i < n;                              // n is a multiple of 4
    // Nothing of this kernel may run ahead of the kernels before it: the epoch below is written by the previous
    // all-reduce, which is only known to be complete once the kernel directly ahead (which waited for its own
    // predecessor in turn) is complete.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) e_s = epoch[c] + 1u;
    __syncthreads();
    const uint32_t e = e_s, par = e & 1u;
    // 1. this rank's values to every rank
    if (valid) {
        const float4 v = *(const float4 *)(x + i);
#pragma unroll
        for (int r = 0; r < W; ++r) *(float4 *)(peers.slots[r] + ((size_t)(par * W + rank)) * n_max + i) = v;
    }
    // 2. the stores are visible system-wide before the flags that announce them
    __threadfence_system();
    __syncthreads();
    if (tid < (uint32_t)W) {
        volatile uint32_t *f = peers.flags[tid] + (size_t)rank * ctas + c;
        *f = e;
    }
    // 3. wait for every sender's flag in this rank's own buffer
    if (tid < (uint32_t)W) {
        volatile uint32_t *f = peers.flags[rank] + (size_t)tid * ctas + c;
        // once a wait has given up, later calls give up quickly too instead of stalling for the full limit each time
        const uint32_t limit = *(volatile uint32_t *)err ? 64u : kArSpinLimit;
        uint32_t polls = 0;
        while ((int32_t)(*f - e) < 0) {
            __nanosleep(32);
            if (++polls > limit) {
                *err = 1u + tid;                           // sender tid never arrived: the result is wrong, not a hang
                break;
            }
        }
    }
    __syncthreads();
    __threadfence_system();
    // 4. sum in rank order
    if (valid) {
        const float *mine = peers.slots[rank] + (size_t)par * W * n_max + i;
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < W; ++r) {
            const float4 v = __ldcv((const float4 *)(mine + (size_t)r * n_max));      // written by a peer: never cached
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        float o[4] = {s.x, s.y, s.z, s.w};
        if (y_f32) {
#pragma unroll
            for (int k = 0; k < 4; ++k) ((float *)y)[i + k] = bias ? o[k] + __bfloat162float(bias[i + k]) : o[k];
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                __nv_bfloat16 h = __float2bfloat16_rn(o[k]);
                if (bias) h = __hadd(h, bias[i + k]);
                ((__nv_bfloat16 *)y)[i + k] = h;
            }
        }
    }
    if (tid == 0) epoch[c] = e;
}

}  // namespace ixb
