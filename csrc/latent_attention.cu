// Latent attention: every token caches ONE row [latent c (kv_rank) | rotated key part (rot)] shared by all heads.
// Queries are pulled through the key up-projection beforehand (q_abs = W_uk^T q_unrotated, a batched GEMM), so a
// score is q_abs . c + q_rot . k_rot and the weighted sum runs over the latents themselves; the value up-projection
// follows as another batched GEMM.  Sliding window, fp32 scores / softmax / accumulation.
#include "common.h"
#include "ptx.cuh"

namespace b200 {

__device__ __forceinline__ void* latent_row(const b200_latent_args& a, int t, int p) {
    const size_t row_bytes = (size_t)a.row_elems * (a.cache_dtype == B200_F32 ? 4 : 2);
    char* base = a.kv_ptrs ? reinterpret_cast<char*>(a.kv_ptrs[(size_t)t * a.kv_ptr_stride]) : static_cast<char*>(a.cache);
    return base + (size_t)p * row_bytes;
}

// ------------------------------------------------------------------ rotary + cache append (one block per token)
__global__ void __launch_bounds__(128) latent_rope_append_kernel(b200_latent_args a) {
    extern __shared__ float cs[];          // [half] cos, [half] sin
    __shared__ float red[4];
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int t = blockIdx.x, tid = threadIdx.x;
    const int p = a.pos ? a.pos[t] : a.pos0 + t;
    const int half = a.rot_dims / 2;
    float* sn = cs + half;
    for (int i = tid; i < half; i += blockDim.x) {
        double s, c;
        sincos((double)p * a.inv_freq[i], &s, &c);
        cs[i] = (float)c;
        sn[i] = (float)s;
    }
    __syncthreads();
    float* row = a.proj + (size_t)t * a.ldp;
    const int hd = a.dim + a.rot;
    for (int idx = tid; idx < a.heads * half; idx += blockDim.x) {
        const int h = idx / half, i = idx - h * half;
        float* q = row + a.q_off + h * hd + a.dim;
        const float u = q[i], v = q[i + half];
        q[i] = u * cs[i] - v * sn[i];
        q[i + half] = v * cs[i] + u * sn[i];
    }
    if (a.kv_off < 0) return;
    const float* src = row + a.kv_off;
    float ss = 0.f;
    for (int c = tid; c < a.kv_rank; c += blockDim.x) ss += src[c] * src[c];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    const float rstd = 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)a.kv_rank + a.eps);
    void* dst = latent_row(a, t, p);
    const bool f32 = a.cache_dtype == B200_F32;
    const int bf = a.cache_dtype == B200_BF16;
    auto put = [&](int c, float v) {
        if (f32)
            static_cast<float*>(dst)[c] = v;
        else
            static_cast<uint16_t*>(dst)[c] = float_to_h16(v, bf);
    };
    for (int c = tid; c < a.kv_rank; c += blockDim.x) put(c, src[c] * rstd * a.c_gain[c]);
    const float* kr = src + a.kv_rank;
    for (int i = tid; i < half; i += blockDim.x) {
        const float u = kr[i], v = kr[i + half];
        put(a.kv_rank + i, u * cs[i] - v * sn[i]);
        put(a.kv_rank + i + half, v * cs[i] + u * sn[i]);
    }
    for (int c = a.rot_dims + tid; c < a.rot; c += blockDim.x) put(a.kv_rank + c, kr[c]);
}

// ------------------------------------------------------------------ attention over the cached rows
constexpr int kHeadsPerBlock = 8;
constexpr int kChunk = 32;

// splits > 1 (decode sizes): blockIdx.z takes a contiguous share of the window's keys and leaves its unnormalised
// (acc, m, l) in `part` [T][heads][splits][kv_rank + 2]; latent_merge_kernel combines the shares in index order.
template <int NPER>
__global__ void __launch_bounds__(256) latent_attn_kernel(b200_latent_args a, int splits, float* __restrict__ part) {
    extern __shared__ float sm[];
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int R = a.kv_rank, rot = a.rot, E = R + rot;
    const int ldk = E | 1;                                   // odd row stride: lane j reads row j without conflicts
    float* qs = sm;                                          // [8][E]
    float* kc = sm + kHeadsPerBlock * E;                     // [32][ldk]
    const int h = blockIdx.y * kHeadsPerBlock + warp;
    const bool live = h < a.heads;
    const int p = a.pos ? a.pos[t] : a.pos0 + t;
    int lo = p - a.window + 1 > 0 ? p - a.window + 1 : 0;
    int hi = p;                                              // last key of this block's share
    if (splits > 1) {
        const int per = ((p - lo + splits) / splits + kChunk - 1) / kChunk * kChunk;
        lo += blockIdx.z * per;
        hi = lo + per - 1 < p ? lo + per - 1 : p;
    }
    if (live) {
        const float* qa = a.q_abs + (size_t)t * a.ldqa + (size_t)h * R;
        const float* qr = a.proj + (size_t)t * a.ldp + a.q_off + h * (a.dim + rot) + a.dim;
        for (int d = lane; d < R; d += 32) qs[warp * E + d] = qa[d];
        for (int d = lane; d < rot; d += 32) qs[warp * E + R + d] = qr[d];
    }
    const bool f32 = a.cache_dtype == B200_F32;
    const int bf = a.cache_dtype == B200_BF16;
    const char* base = static_cast<const char*>(latent_row(a, t, 0));
    const bool vec16 = !f32 && E % 8 == 0 && a.row_elems % 8 == 0 && (reinterpret_cast<uintptr_t>(base) & 15) == 0;
    float m = -INFINITY, l = 0.f, acc[NPER];
#pragma unroll
    for (int i = 0; i < NPER; ++i) acc[i] = 0.f;
    for (int j0 = lo; j0 <= hi; j0 += kChunk) {
        const int n = hi - j0 + 1 < kChunk ? hi - j0 + 1 : kChunk;
        __syncthreads();                                     // previous chunk fully consumed (and qs written)
        if (vec16) {          // 16-byte loads, several in flight per thread (a dependent 2-byte load per element is
            const int cpr = E / 8;   // latency-bound: ~70 us per 32 keys on a cold cache)
#pragma unroll 4
            for (int e = tid; e < n * cpr; e += 256) {
                const int j = e / cpr, d = (e - j * cpr) * 8;
                const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + (size_t)(j0 + j) * a.row_elems + d);
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
                float* dst = kc + j * ldk + d;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    dst[2 * i] = h16_to_float((uint16_t)(w[i] & 0xffff), bf);
                    dst[2 * i + 1] = h16_to_float((uint16_t)(w[i] >> 16), bf);
                }
            }
        } else {
#pragma unroll 4
            for (int e = tid; e < n * E; e += 256) {
                const int j = e / E, d = e - j * E;
                const size_t g = (size_t)(j0 + j) * a.row_elems + d;
                kc[j * ldk + d] = f32 ? reinterpret_cast<const float*>(base)[g]
                                      : h16_to_float(reinterpret_cast<const uint16_t*>(base)[g], bf);
            }
        }
        __syncthreads();
        if (!live) continue;
        float s = -INFINITY;
        if (lane < n) {
            const float* q = qs + warp * E;
            const float* k = kc + lane * ldk;
            float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;   // four chains: the sum is latency-bound otherwise
            int d = 0;
            for (; d + 4 <= E; d += 4) {
                d0 = fmaf(q[d], k[d], d0);
                d1 = fmaf(q[d + 1], k[d + 1], d1);
                d2 = fmaf(q[d + 2], k[d + 2], d2);
                d3 = fmaf(q[d + 3], k[d + 3], d3);
            }
            for (; d < E; ++d) d0 = fmaf(q[d], k[d], d0);
            s = ((d0 + d1) + (d2 + d3)) * a.scale;
        }
        float cm = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
        const float mn = fmaxf(m, cm);                       // finite: every chunk holds at least one key
        const float alpha = expf(m - mn);                    // first chunk: exp(-inf) = 0
        const float pj = lane < n ? expf(s - mn) : 0.f;
        float ps = pj;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        l = l * alpha + ps;
        m = mn;
#pragma unroll
        for (int i = 0; i < NPER; ++i) acc[i] *= alpha;
        for (int j = 0; j < n; ++j) {
            const float w = __shfl_sync(0xffffffffu, pj, j);
            const float* k = kc + j * ldk;
#pragma unroll
            for (int i = 0; i < NPER; ++i) {
                const int d = lane + 32 * i;
                if (d < R) acc[i] = fmaf(w, k[d], acc[i]);
            }
        }
    }
    if (!live) return;
    if (splits > 1) {                                        // (a share without keys leaves m = -inf, l = 0)
        float* o = part + (((size_t)t * a.heads + h) * splits + blockIdx.z) * (R + 2);
#pragma unroll
        for (int i = 0; i < NPER; ++i) {
            const int d = lane + 32 * i;
            if (d < R) o[d] = acc[i];
        }
        if (lane == 0) {
            o[R] = m;
            o[R + 1] = l;
        }
        return;
    }
    float* o = a.out + (size_t)t * a.ldout + (size_t)h * R;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
        const int d = lane + 32 * i;
        if (d < R) o[d] = acc[i] * inv;
    }
}

// One warp per (token, head, 32 output columns): the shares' (acc, m, l) merged in index order, then normalised.
// Lane s holds the weight exp(m_s - m) of share s (splits <= 32).
__global__ void __launch_bounds__(128) latent_merge_kernel(const float* __restrict__ part, float* __restrict__ out, int ldout,
                                                          int T, int heads, int R, int splits) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int slices = (R + 31) / 32;
    const int w = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= T * heads * slices) return;
    const int th = w / slices, d = (w - th * slices) * 32 + lane;
    const int t = th / heads, h = th - t * heads;
    const float* p = part + (size_t)th * splits * (R + 2);
    const float ms = lane < splits ? p[(size_t)lane * (R + 2) + R] : -INFINITY;
    const float ls = lane < splits ? p[(size_t)lane * (R + 2) + R + 1] : 0.f;
    float m = ms;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float ws = ms > -INFINITY ? expf(ms - m) : 0.f;
    float l = 0.f, acc = 0.f;
    for (int s = 0; s < splits; ++s) {                                               // index order
        const float wv = __shfl_sync(0xffffffffu, ws, s);
        l += __shfl_sync(0xffffffffu, ls, s) * wv;
        if (d < R && wv != 0.f) acc += wv * p[(size_t)s * (R + 2) + d];
    }
    if (d < R) out[(size_t)t * ldout + (size_t)h * R + d] = acc / l;
}

template <int NPER>
static int launch_attn(const b200_latent_args* a, size_t smem, cudaStream_t s, int splits, float* part) {
    if (smem > 48 * 1024)
        B200_CUDA_CHECK(cudaFuncSetAttribute(latent_attn_kernel<NPER>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(a->T, (a->heads + kHeadsPerBlock - 1) / kHeadsPerBlock, splits);
    B200_CUDA_CHECK(launch(latent_attn_kernel<NPER>, grid, dim3(256), smem, s, a->pdl != 0, *a, splits, part));
    if (splits > 1)
        B200_CUDA_CHECK(launch(latent_merge_kernel, dim3((a->T * a->heads * ((a->kv_rank + 31) / 32) + 3) / 4), dim3(128), 0, s, a->pdl != 0,
                               (const float*)part, a->out, a->ldout, a->T, a->heads, a->kv_rank, splits));
    return B200_OK;
}

}  // namespace b200

using namespace b200;

static int check_latent(const b200_latent_args* a, const char* who) {
    if (!a || !a->proj || (!a->cache && !a->kv_ptrs)) return fail(B200_EINVAL, "%s: null pointer argument", who);
    if (a->T <= 0 || a->heads <= 0 || a->dim < 0 || a->rot < 0 || a->kv_rank <= 0 || a->rot_dims > a->rot || (a->rot_dims & 1) ||
        a->row_elems < a->kv_rank + a->rot)
        return fail(B200_EINVAL, "%s: bad sizes (heads %d dim %d rot %d rot_dims %d kv_rank %d row %d)", who, a->heads, a->dim,
                    a->rot, a->rot_dims, a->kv_rank, a->row_elems);
    if (a->cache_dtype != B200_F32 && a->cache_dtype != B200_BF16 && a->cache_dtype != B200_F16)
        return fail(B200_EINVAL, "%s: bad cache element type %d", who, a->cache_dtype);
    return B200_OK;
}

extern "C" int b200_latent_rope_append(const b200_latent_args* a, void* stream) {
    if (int rc = check_latent(a, "b200_latent_rope_append")) return rc;
    if (a->rot_dims > 0 && !a->inv_freq) return fail(B200_EINVAL, "b200_latent_rope_append: rotation without inv_freq");
    if (a->kv_off >= 0 && !a->c_gain) return fail(B200_EINVAL, "b200_latent_rope_append: cache append without the latent's gain");
    const size_t smem = (size_t)(a->rot_dims > 0 ? a->rot_dims : 2) * sizeof(float);
    B200_CUDA_CHECK(launch(latent_rope_append_kernel, dim3(a->T), dim3(128), smem, static_cast<cudaStream_t>(stream), a->pdl != 0, *a));
    return B200_OK;
}

extern "C" int64_t b200_latent_attn_scratch_bytes(int32_t T, int32_t heads, int32_t kv_rank, int32_t splits) {
    return (int64_t)T * heads * splits * (kv_rank + 2) * (int64_t)sizeof(float);
}

extern "C" int b200_latent_attn(const b200_latent_args* a, void* stream) {
    return b200_latent_attn_split(a, 1, nullptr, stream);
}

extern "C" int b200_latent_attn_split(const b200_latent_args* a, int32_t splits, float* scratch, void* stream) {
    if (int rc = check_latent(a, "b200_latent_attn")) return rc;
    if (splits < 1 || splits > 32 || (splits > 1 && !scratch)) return fail(B200_EINVAL, "b200_latent_attn: bad splits %d", splits);
    if (!a->q_abs || !a->out || a->window <= 0) return fail(B200_EINVAL, "b200_latent_attn: q_abs / out / window missing");
    const int E = a->kv_rank + a->rot;
    const size_t smem = ((size_t)kHeadsPerBlock * E + (size_t)kChunk * (E | 1)) * sizeof(float);
    if (smem > 220 * 1024) return fail(B200_ELIMIT, "b200_latent_attn: kv_rank + rot = %d exceeds shared memory", E);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int nper = (a->kv_rank + 31) / 32;
    if (nper <= 1) return launch_attn<1>(a, smem, s, splits, scratch);
    if (nper <= 2) return launch_attn<2>(a, smem, s, splits, scratch);
    if (nper <= 4) return launch_attn<4>(a, smem, s, splits, scratch);
    if (nper <= 8) return launch_attn<8>(a, smem, s, splits, scratch);
    if (nper <= 16) return launch_attn<16>(a, smem, s, splits, scratch);
    if (nper <= 32) return launch_attn<32>(a, smem, s, splits, scratch);
    return fail(B200_ELIMIT, "b200_latent_attn: kv_rank %d > 1024", a->kv_rank);
}
