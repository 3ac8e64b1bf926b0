// Elementwise kernels of designs that keep the residual stream in fp32: embedding gather to fp32, residual update
// fused with the RMS norm that follows it, and the clamped gated unit of a feed-forward layer.
#include "common.h"
#include "ptx.cuh"

namespace b200 {

__device__ __forceinline__ float load_elem(const void* p, size_t i, int dtype) {
    if (dtype == B200_F32) return static_cast<const float*>(p)[i];
    return h16_to_float(static_cast<const uint16_t*>(p)[i], dtype == B200_BF16);
}
__device__ __forceinline__ void store_elem(void* p, size_t i, float v, int dtype) {
    if (dtype == B200_F32)
        static_cast<float*>(p)[i] = v;
    else
        static_cast<uint16_t*>(p)[i] = float_to_h16(v, dtype == B200_BF16);
}

// ------------------------------------------------------------------ embedding -> fp32
__global__ void __launch_bounds__(128) embed_f32_kernel(const long long* __restrict__ ids, const void* __restrict__ table,
                                                       int dtype, float* __restrict__ out, int T, int width, int ldo,
                                                       int vocab) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    if (t >= T) return;
    long long id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    for (int c = threadIdx.x; c < width; c += blockDim.x) out[(size_t)t * ldo + c] = load_elem(table, (size_t)id * width + c, dtype);
}

__global__ void __launch_bounds__(128) embed_pos_f32_kernel(const long long* __restrict__ ids, const void* __restrict__ table,
                                                           const void* __restrict__ pos_table, int dtype,
                                                           const int* __restrict__ pos, int pos0, float* __restrict__ out,
                                                           int T, int width, int ldo, int vocab, int max_pos) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    if (t >= T) return;
    long long id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    int p = pos ? pos[t] : pos0 + t;
    p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);
    for (int c = threadIdx.x; c < width; c += blockDim.x)
        out[(size_t)t * ldo + c] = load_elem(table, (size_t)id * width + c, dtype) + load_elem(pos_table, (size_t)p * width + c, dtype);
}

// ------------------------------------------------------------------ residual update + RMS norm
// One block per token.  The updated row is kept in shared memory between the two passes.
__global__ void __launch_bounds__(256) add_rms_norm_kernel(b200_add_norm_args a, int vec) {
    extern __shared__ __align__(16) float row[];
    __shared__ float red[8];
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    float* x = a.x + (size_t)t * a.ldx;
    float ss = 0.f;
    if (vec) {      // four columns per thread and pass (16-byte accesses); the sums keep their order per column
        for (int c = threadIdx.x * 4; c < a.width; c += blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(x + c);
            float4 add = make_float4(0.f, 0.f, 0.f, 0.f);
            bool any = false;
            if (a.add_a) {
                const float4 y = *reinterpret_cast<const float4*>(a.add_a + (size_t)t * a.lda + c);
                add.x += y.x, add.y += y.y, add.z += y.z, add.w += y.w;
                any = true;
            }
            if (a.add_b) {
                const float4 y = *reinterpret_cast<const float4*>(a.add_b + (size_t)t * a.ldb + c);
                add.x += y.x, add.y += y.y, add.z += y.z, add.w += y.w;
                any = true;
            }
            if (a.pair_y) {
                float4 m = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int k = 0; k < a.top; ++k) {
                    const size_t p = (size_t)t * a.top + k;
                    const float4 y = *reinterpret_cast<const float4*>(a.pair_y + p * a.ldp + c);
                    const float w = a.pair_w ? a.pair_w[p] : 1.0f;
                    if (a.pair_w)
                        m.x += w * y.x, m.y += w * y.y, m.z += w * y.z, m.w += w * y.w;
                    else
                        m.x += y.x, m.y += y.y, m.z += y.z, m.w += y.w;
                }
                add.x += m.x, add.y += m.y, add.z += m.z, add.w += m.w;
                any = true;
            }
            if (any) {
                v.x += a.add_scale * add.x, v.y += a.add_scale * add.y, v.z += a.add_scale * add.z, v.w += a.add_scale * add.w;
                *reinterpret_cast<float4*>(x + c) = v;
            }
            *reinterpret_cast<float4*>(row + c) = v;
            ss += v.x * v.x;
            ss += v.y * v.y;
            ss += v.z * v.z;
            ss += v.w * v.w;
        }
    } else
    for (int c = threadIdx.x; c < a.width; c += blockDim.x) {
        float v = x[c];
        float add = 0.f;
        bool any = false;
        if (a.add_a) { add += a.add_a[(size_t)t * a.lda + c]; any = true; }
        if (a.add_b) { add += a.add_b[(size_t)t * a.ldb + c]; any = true; }
        if (a.pair_y) {
            float m = 0.f;
            for (int k = 0; k < a.top; ++k) {
                const size_t p = (size_t)t * a.top + k;
                const float y = a.pair_y[p * a.ldp + c];
                m += a.pair_w ? a.pair_w[p] * y : y;
            }
            add += m;
            any = true;
        }
        if (any) {
            v += a.add_scale * add;
            x[c] = v;
        }
        row[c] = v;
        ss += v * v;
    }
    if (!a.out) return;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += red[w];
    const float rstd = 1.0f / sqrtf(tot / (float)a.width + a.eps);
    if (vec && a.out_dtype != B200_F32) {
        const int bf = a.out_dtype == B200_BF16;
        for (int c = threadIdx.x * 4; c < a.width; c += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(row + c);
            const float4 g = *reinterpret_cast<const float4*>(a.gain + c);
            uint2 o;
            o.x = (uint32_t)float_to_h16(v.x * rstd * (a.gain_offset + g.x), bf) | ((uint32_t)float_to_h16(v.y * rstd * (a.gain_offset + g.y), bf) << 16);
            o.y = (uint32_t)float_to_h16(v.z * rstd * (a.gain_offset + g.z), bf) | ((uint32_t)float_to_h16(v.w * rstd * (a.gain_offset + g.w), bf) << 16);
            *reinterpret_cast<uint2*>(static_cast<uint16_t*>(a.out) + (size_t)t * a.ldo + c) = o;
        }
        return;
    }
    for (int c = threadIdx.x; c < a.width; c += blockDim.x)
        store_elem(a.out, (size_t)t * a.ldo + c, row[c] * rstd * (a.gain_offset + a.gain[c]), a.out_dtype);
}

// ------------------------------------------------------------------ clamped gated unit
__global__ void __launch_bounds__(256) glu_clamp_kernel(const float* __restrict__ gate, const float* __restrict__ up, int ld,
                                                       void* __restrict__ act, int ldo, int out_dtype, int T, int ff,
                                                       float limit, float alpha, float up_shift) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const size_t n = (size_t)T * ff;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / ff), c = (int)(i - (size_t)t * ff);
        float g = gate[(size_t)t * ld + c], u = up[(size_t)t * ld + c];
        if (limit > 0.f) {
            g = fminf(g, limit);
            u = fminf(fmaxf(u, -limit), limit);
        }
        const float y = g / (1.0f + expf(-alpha * g)) * (u + up_shift);
        store_elem(act, (size_t)t * ldo + c, y, out_dtype);
    }
}

// ------------------------------------------------------------------ piecewise activation with two learned numbers
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

__global__ void __launch_bounds__(256) xielu_kernel(const float* __restrict__ z, int ld, const float* __restrict__ params,
                                                   float lin, float neg_base, void* __restrict__ act, int ldo, int out_dtype,
                                                   int T, int ff, int vec) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const float ap = softplus_f(params[0]), an = neg_base + softplus_f(params[1]);
    const size_t n = (size_t)T * ff;
    if (vec) {      // four values per thread: 16-byte loads, 8-byte (16-bit output) or 16-byte stores
        const int q = ff / 4;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)T * q; i += (size_t)gridDim.x * blockDim.x) {
            const int t = (int)(i / q), c = (int)(i - (size_t)t * q) * 4;
            const float4 v = *reinterpret_cast<const float4*>(z + (size_t)t * ld + c);
            float y[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) y[k] = y[k] > 0.f ? fmaf(ap * y[k], y[k], lin * y[k]) : fmaf(an, expm1f(y[k]) - y[k], lin * y[k]);
            if (out_dtype == B200_F32) {
                *reinterpret_cast<float4*>(static_cast<float*>(act) + (size_t)t * ldo + c) = make_float4(y[0], y[1], y[2], y[3]);
            } else {
                const int bf = out_dtype == B200_BF16;
                uint2 o;
                o.x = (uint32_t)float_to_h16(y[0], bf) | ((uint32_t)float_to_h16(y[1], bf) << 16);
                o.y = (uint32_t)float_to_h16(y[2], bf) | ((uint32_t)float_to_h16(y[3], bf) << 16);
                *reinterpret_cast<uint2*>(static_cast<uint16_t*>(act) + (size_t)t * ldo + c) = o;
            }
        }
        return;
    }
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / ff), c = (int)(i - (size_t)t * ff);
        const float v = z[(size_t)t * ld + c];
        const float y = v > 0.f ? fmaf(ap * v, v, lin * v) : fmaf(an, expm1f(v) - v, lin * v);
        store_elem(act, (size_t)t * ldo + c, y, out_dtype);
    }
}

// ------------------------------------------------------------------ gated RMS norm per head (one warp per token and head)
__global__ void __launch_bounds__(128) gated_head_norm_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ gate,
                                                             int ldg, const float* __restrict__ gain, void* __restrict__ out,
                                                             int ldout, int out_dtype, int T, int heads, int vdim, float eps) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int w = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= T * heads) return;
    const int t = w / heads, h = w - t * heads;
    const float* src = o + (size_t)t * ldo + (size_t)h * vdim;
    const float* g = gate + (size_t)t * ldg + (size_t)h * vdim;
    float ss = 0.f;
    for (int d = lane; d < vdim; d += 32) ss = fmaf(src[d], src[d], ss);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
    const float rstd = 1.0f / sqrtf(ss / (float)vdim + eps);
    for (int d = lane; d < vdim; d += 32) {
        const float z = g[d];
        store_elem(out, (size_t)t * ldout + (size_t)h * vdim + d, src[d] * rstd * gain[d] * (z / (1.0f + expf(-z))), out_dtype);
    }
}

// ------------------------------------------------------------------ one sigmoid gate per token and head, in place
__global__ void __launch_bounds__(256) head_gate_kernel(void* __restrict__ x, int ldx, int dtype, const float* __restrict__ gate,
                                                       int ldg, int T, int heads, int vdim, int vec) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const size_t n = (size_t)T * heads * vdim;
    if (vec) {      // 16-bit values, eight per thread (they share a head)
        const int per_row = heads * vdim / 8, bf = dtype == B200_BF16;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n / 8; i += (size_t)gridDim.x * blockDim.x) {
            const int t = (int)(i / per_row), c = (int)(i - (size_t)t * per_row) * 8, h = c / vdim;
            const float g = 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + h]));
            uint4* p = reinterpret_cast<uint4*>(static_cast<uint16_t*>(x) + (size_t)t * ldx + c);
            uint4 v = *p;
            uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k)
                w[k] = (uint32_t)float_to_h16(h16_to_float((uint16_t)(w[k] & 0xffff), bf) * g, bf) |
                       ((uint32_t)float_to_h16(h16_to_float((uint16_t)(w[k] >> 16), bf) * g, bf) << 16);
            *p = make_uint4(w[0], w[1], w[2], w[3]);
        }
        return;
    }
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / ((size_t)heads * vdim)), c = (int)(i - (size_t)t * heads * vdim), h = c / vdim;
        const float g = 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + h]));
        store_elem(x, (size_t)t * ldx + c, load_elem(x, (size_t)t * ldx + c, dtype) * g, dtype);
    }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_head_gate(void* x, int32_t ldx, int32_t dtype, const float* gate, int32_t ldg, int32_t T, int32_t heads,
                              int32_t vdim, int32_t pdl, void* stream) {
    if (!x || !gate || T <= 0 || heads <= 0 || vdim <= 0) return fail(B200_EINVAL, "b200_head_gate: bad argument");
    const int vec = (dtype != B200_F32 && vdim % 8 == 0 && ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) ? 1 : 0;
    const size_t n = (size_t)T * heads * vdim / (vec ? 8 : 1);
    const int blocks = (int)((n + 255) / 256 < 8192 ? (n + 255) / 256 : 8192);
    B200_CUDA_CHECK(launch(head_gate_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream), pdl != 0, x, ldx, dtype,
                           gate, ldg, T, heads, vdim, vec));
    return B200_OK;
}

extern "C" int b200_embed_pos_f32(const void* ids, const void* table, const void* pos_table, int32_t table_dtype,
                                  const int32_t* pos, int32_t pos0, float* out, int32_t T, int32_t width, int32_t ldo,
                                  int32_t vocab, int32_t max_pos, int32_t pdl, void* stream) {
    if (!ids || !table || !pos_table || !out || T <= 0 || width <= 0 || max_pos <= 0)
        return fail(B200_EINVAL, "b200_embed_pos_f32: bad argument");
    B200_CUDA_CHECK(launch(embed_pos_f32_kernel, dim3(T), dim3(128), 0, static_cast<cudaStream_t>(stream), pdl != 0,
                           static_cast<const long long*>(ids), table, pos_table, table_dtype, pos, pos0, out, T, width, ldo,
                           vocab, max_pos));
    return B200_OK;
}

extern "C" int b200_xielu(const float* z, int32_t ld, const float* params, float lin, float neg_base, void* act, int32_t ldo,
                          int32_t out_dtype, int32_t T, int32_t ff, int32_t pdl, void* stream) {
    if (!z || !params || !act || T <= 0 || ff <= 0) return fail(B200_EINVAL, "b200_xielu: bad argument");
    const int vec = (ff % 4 == 0 && ld % 4 == 0 && ldo % 4 == 0 && (reinterpret_cast<uintptr_t>(z) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(act) & 15) == 0) ? 1 : 0;
    const size_t n = (size_t)T * ff / (vec ? 4 : 1);
    const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    B200_CUDA_CHECK(launch(xielu_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream), pdl != 0, z, ld, params,
                           lin, neg_base, act, ldo, out_dtype, T, ff, vec));
    return B200_OK;
}

extern "C" int b200_gated_head_norm(const float* o, int32_t ldo, const float* gate, int32_t ldg, const float* gain, void* out,
                                    int32_t ldout, int32_t out_dtype, int32_t T, int32_t heads, int32_t vdim, float eps,
                                    int32_t pdl, void* stream) {
    if (!o || !gate || !gain || !out || T <= 0 || heads <= 0 || vdim <= 0)
        return fail(B200_EINVAL, "b200_gated_head_norm: bad argument");
    B200_CUDA_CHECK(launch(gated_head_norm_kernel, dim3((T * heads + 3) / 4), dim3(128), 0, static_cast<cudaStream_t>(stream),
                           pdl != 0, o, ldo, gate, ldg, gain, out, ldout, out_dtype, T, heads, vdim, eps));
    return B200_OK;
}

extern "C" int b200_embed_f32(const void* ids, const void* table, int32_t table_dtype, float* out, int32_t T, int32_t width,
                              int32_t ldo, int32_t vocab, int32_t pdl, void* stream) {
    if (!ids || !table || !out || T <= 0 || width <= 0) return fail(B200_EINVAL, "b200_embed_f32: bad argument");
    B200_CUDA_CHECK(launch(embed_f32_kernel, dim3(T), dim3(128), 0, static_cast<cudaStream_t>(stream), pdl != 0,
                           static_cast<const long long*>(ids), table, table_dtype, out, T, width, ldo, vocab));
    return B200_OK;
}

extern "C" int b200_add_rms_norm(const b200_add_norm_args* a, void* stream) {
    if (!a || !a->x || a->T <= 0 || a->width <= 0) return fail(B200_EINVAL, "b200_add_rms_norm: bad argument");
    if (a->out && !a->gain) return fail(B200_EINVAL, "b200_add_rms_norm: out without gain");
    const size_t smem = (size_t)a->width * sizeof(float);
    if (smem > 200 * 1024) return fail(B200_ELIMIT, "b200_add_rms_norm: width %d exceeds the row buffer", a->width);
    if (smem > 48 * 1024)
        B200_CUDA_CHECK(cudaFuncSetAttribute(add_rms_norm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const int vec = (a->width % 4 == 0 && a->ldx % 4 == 0 && al16(a->x) && (!a->add_a || (a->lda % 4 == 0 && al16(a->add_a))) &&
                     (!a->add_b || (a->ldb % 4 == 0 && al16(a->add_b))) && (!a->pair_y || (a->ldp % 4 == 0 && al16(a->pair_y))) &&
                     (!a->out || (al16(a->gain) && a->ldo % 4 == 0 && (reinterpret_cast<uintptr_t>(a->out) & 7) == 0))) ? 1 : 0;
    B200_CUDA_CHECK(launch(add_rms_norm_kernel, dim3(a->T), dim3(256), smem, static_cast<cudaStream_t>(stream), a->pdl != 0, *a, vec));
    return B200_OK;
}

extern "C" int b200_glu_clamp(const float* gate, const float* up, int32_t ld, void* act, int32_t ldo, int32_t out_dtype,
                              int32_t T, int32_t ff, float limit, float alpha, float up_shift, int32_t pdl, void* stream) {
    if (!gate || !up || !act || T <= 0 || ff <= 0) return fail(B200_EINVAL, "b200_glu_clamp: bad argument");
    const size_t n = (size_t)T * ff;
    const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    B200_CUDA_CHECK(launch(glu_clamp_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream), pdl != 0, gate, up,
                           ld, act, ldo, out_dtype, T, ff, limit, alpha, up_shift));
    return B200_OK;
}
