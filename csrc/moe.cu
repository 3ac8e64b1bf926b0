// Mixture of experts, the parts around the expert GEMMs: the router (softmax over all experts, group-limited choice,
// top-k) and the plan that sorts (token, slot) pairs by expert for the grouped GEMM (b200_gemm_simt with group_off).
#include "common.h"
#include "ptx.cuh"

namespace b200 {

// lowest index among the lanes holding the largest value
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) {
            v = ov;
            i = oi;
        }
    }
}

__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, int ld, int T, int E, int G, int keep,
                                                       int top, int renorm, int* __restrict__ ids, float* __restrict__ wts) {
    extern __shared__ float sm[];
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= T) return;
    float* sc = sm + (size_t)warp * (E + G);       // scores; chosen ones are overwritten with -1
    float* gs = sc + E;                            // group scores; -2 = group not kept, -1 while choosing
    const float* z = logits + (size_t)t * ld;
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
        const float v = expf(z[e] - mx);
        sc[e] = v;
        sum += v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32) sc[e] *= inv;
    __syncwarp();
    const int per = E / G;
    const bool limited = G > 1 && keep < G;
    if (limited) {
        for (int g = lane; g < G; g += 32) {
            float v = sc[g * per];
            for (int e = 1; e < per; ++e) v = fmaxf(v, sc[g * per + e]);
            gs[g] = v;
        }
        __syncwarp();
        for (int k = 0; k < keep; ++k) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            for (int g = lane; g < G; g += 32)
                if (gs[g] >= 0.f && (gs[g] > bv)) {
                    bv = gs[g];
                    bi = g;
                }
            warp_argmax(bv, bi);
            if (lane == 0 && bi < G) gs[bi] = -1.f;          // kept
            __syncwarp();
        }
        for (int g = lane; g < G; g += 32) gs[g] = gs[g] == -1.f ? 1.f : 0.f;
        __syncwarp();
    }
    float wsum = 0.f;
    for (int k = 0; k < top; ++k) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            if (limited && gs[e / per] == 0.f) continue;
            const float v = sc[e];
            if (v >= 0.f && v > bv) {
                bv = v;
                bi = e;
            }
        }
        warp_argmax(bv, bi);
        if (lane == 0) {
            const int e = bi < E ? bi : 0;
            ids[(size_t)t * top + k] = e;
            wts[(size_t)t * top + k] = bi < E ? bv : 0.f;
            if (bi < E) sc[bi] = -1.f;
        }
        wsum += bi < E ? bv : 0.f;
        __syncwarp();
    }
    if (renorm && lane == 0 && wsum > 0.f)
        for (int k = 0; k < top; ++k) wts[(size_t)t * top + k] /= wsum;
}

__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* __restrict__ ids, int n_pairs, int top, int E,
                                                       int* __restrict__ group_off, int* __restrict__ row_pair,
                                                       int* __restrict__ row_token) {
    extern __shared__ int si[];                    // [E] counts -> cursors, [E + 1] offsets
    int* cnt = si;
    int* off = si + E;
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&cnt[ids[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            off[e] = run;
            run += cnt[e];
        }
        off[E] = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) group_off[e] = off[e];
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = ids[i];
        const int r = off[e] + atomicAdd(&cnt[e], 1);
        row_pair[r] = i;
        row_token[r] = i / top;
    }
}

// act[t, e * ff + j] *= weight of expert e for token t (0 when e was not chosen): turns the outputs of ALL experts'
// gated units into the operand of one down-projection over the concatenated experts.
__global__ void __launch_bounds__(256) moe_scale_kernel(uint16_t* __restrict__ act, int ld, const int* __restrict__ ids,
                                                       const float* __restrict__ wts, int T, int E, int ff, int top, int is_bf16) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int t = blockIdx.y;
    const int n = E * ff;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int e = i / ff;
        float w = 0.f;
        for (int k = 0; k < top; ++k)
            if (ids[(size_t)t * top + k] == e) w += wts[(size_t)t * top + k];
        uint16_t* p = act + (size_t)t * ld + i;
        *p = w == 0.f ? (uint16_t)0 : float_to_h16(h16_to_float(*p, is_bf16) * w, is_bf16);
    }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_moe_scale(void* act, int32_t ld, int32_t dtype, const int32_t* ids, const float* weights, int32_t T,
                              int32_t experts, int32_t ff, int32_t top, int32_t pdl, void* stream) {
    if (!act || !ids || !weights || T <= 0 || experts <= 0 || ff <= 0 || top <= 0 || (dtype != B200_F16 && dtype != B200_BF16))
        return fail(B200_EINVAL, "b200_moe_scale: bad argument");
    const int n = experts * ff;
    dim3 grid((n + 1023) / 1024 < 64 ? (n + 1023) / 1024 : 64, T);
    if (T > 65535) return fail(B200_ELIMIT, "b200_moe_scale: T %d", T);
    B200_CUDA_CHECK(launch(moe_scale_kernel, grid, dim3(256), 0, static_cast<cudaStream_t>(stream), pdl != 0,
                           static_cast<uint16_t*>(act), ld, ids, weights, T, experts, ff, top, dtype == B200_BF16 ? 1 : 0));
    return B200_OK;
}

extern "C" int b200_moe_route(const float* logits, int32_t ld, int32_t T, int32_t experts, int32_t groups, int32_t keep,
                              int32_t top, int32_t renorm, int32_t* ids, float* weights, int32_t pdl, void* stream) {
    if (!logits || !ids || !weights || T <= 0) return fail(B200_EINVAL, "b200_moe_route: bad argument");
    if (groups < 1) groups = 1;
    if (experts <= 0 || top <= 0 || top > experts || experts % groups != 0 || keep < 1 || keep > groups ||
        top > keep * (experts / groups))
        return fail(B200_EINVAL, "b200_moe_route: experts %d groups %d keep %d top %d do not fit together", experts, groups, keep, top);
    const size_t smem = (size_t)4 * (experts + groups) * sizeof(float);
    if (smem > 48 * 1024) return fail(B200_ELIMIT, "b200_moe_route: %d experts exceed the router's shared memory", experts);
    B200_CUDA_CHECK(launch(moe_route_kernel, dim3((T + 3) / 4), dim3(128), smem, static_cast<cudaStream_t>(stream), pdl != 0,
                           logits, ld, T, experts, groups, keep, top, renorm, ids, weights));
    return B200_OK;
}

extern "C" int b200_moe_plan(const int32_t* ids, int32_t T, int32_t top, int32_t experts, int32_t* group_off, int32_t* row_pair,
                             int32_t* row_token, int32_t pdl, void* stream) {
    if (!ids || !group_off || !row_pair || !row_token || T <= 0 || top <= 0 || experts <= 0)
        return fail(B200_EINVAL, "b200_moe_plan: bad argument");
    const size_t smem = (size_t)(2 * experts + 1) * sizeof(int);
    if (smem > 48 * 1024) return fail(B200_ELIMIT, "b200_moe_plan: %d experts exceed the plan's shared memory", experts);
    B200_CUDA_CHECK(launch(moe_plan_kernel, dim3(1), dim3(1024), smem, static_cast<cudaStream_t>(stream), pdl != 0, ids, T * top,
                           top, experts, group_off, row_pair, row_token));
    return B200_OK;
}
