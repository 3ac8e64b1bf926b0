// Grouped-query softmax attention without rotation whose denominator carries a sink: normalisation of the projections
// and the cache append (three blocks per token: queries, keys, values), then attention over the cached rows with fp32
// scores, weights and sums (one block per token, head and share of the keys; the shares of a decode step are merged by a
// second launch).
// Cache planes keep all key (value) heads of a position side by side in one row.
#include "common.h"
#include "ptx.cuh"

namespace b200 {

__device__ __forceinline__ char* sink_plane(const b200_sink_attn_args& a, int t, int which) {
    if (a.kv_ptrs) return reinterpret_cast<char*>(a.kv_ptrs[(size_t)t * a.kv_ptr_stride + which]);
    return static_cast<char*>(which ? a.v_cache : a.k_cache);
}

__device__ __forceinline__ float block_sum_256(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();                                  // red may still be read from the previous call
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += red[w];
    return tot;
}

// ------------------------------------------------------------------ norms + cache append
// Three blocks per token: queries, keys, values (each is a chain of dependent passes over its part of the row).
__global__ void __launch_bounds__(256) sink_attn_append_kernel(b200_sink_attn_args a) {
    __shared__ float red[8];
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int p = a.pos ? a.pos[t] : a.pos0 + t;
    float* row = a.proj + (size_t)t * a.ldp;
    const int qn = a.heads * a.dim, kn = a.kv_heads * a.dim, vn = a.kv_heads * a.vdim;
    const bool f32 = a.cache_dtype == B200_F32;
    const int bf = a.cache_dtype == B200_BF16;
    const size_t row_bytes = (size_t)a.row_elems * (f32 ? 4 : 2);
    if (blockIdx.y == 0) {     // queries: bias, one norm over the whole row, score scale and the head's temperature folded in
        float* q = row + a.q_off;
        float ss = 0.f;
        for (int c = tid; c < qn; c += 256) {
            const float v = q[c] + (a.bias ? a.bias[c] : 0.f);
            q[c] = v;
            ss = fmaf(v, v, ss);
        }
        const float rstd = 1.0f / sqrtf(block_sum_256(ss, red) / (float)qn + a.eps);
        for (int c = tid; c < qn; c += 256) {
            const int h = c / a.dim;
            const float v = q[c] * rstd * a.q_gain[c] * (a.scale * (a.temp ? a.temp[h] : 1.0f));
            q[c] = v;
            if (a.q16 && !f32) static_cast<uint16_t*>(a.q16)[(size_t)t * a.ldq16 + c] = float_to_h16(v, bf);
        }
        return;
    }
    if (blockIdx.y == 1) {     // keys
        float* k = row + a.k_off;
        float ss = 0.f;
        for (int c = tid; c < kn; c += 256) {
            const float v = k[c] + (a.bias ? a.bias[qn + c] : 0.f);
            k[c] = v;
            ss = fmaf(v, v, ss);
        }
        const float rstd = 1.0f / sqrtf(block_sum_256(ss, red) / (float)kn + a.eps);
        char* kd = sink_plane(a, t, 0) + (size_t)p * row_bytes;
        for (int c = tid; c < kn; c += 256) {
            const float v = k[c] * rstd * a.k_gain[c];
            if (f32)
                reinterpret_cast<float*>(kd)[c] = v;
            else
                reinterpret_cast<uint16_t*>(kd)[c] = float_to_h16(v, bf);
        }
        return;
    }
    // values: one warp per head at a time
    char* vd = sink_plane(a, t, 1) + (size_t)p * row_bytes;
    const float lam = a.vmix_mode == 2 ? *a.vmix : 0.f;
    for (int g = warp; g < a.kv_heads; g += 8) {
        float* v = row + a.v_off + g * a.vdim;
        float s2 = 0.f;
        for (int d = lane; d < a.vdim; d += 32) {
            const float x = v[d] + (a.bias ? a.bias[qn + kn + g * a.vdim + d] : 0.f);
            v[d] = x;
            s2 = fmaf(x, x, s2);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s2 += __shfl_xor_sync(0xffffffffu, s2, o);
        const float r = 1.0f / sqrtf(s2 / (float)a.vdim + a.eps);
        for (int d = lane; d < a.vdim; d += 32) {
            float x = v[d] * r;
            const int c = g * a.vdim + d;
            if (a.vmix_mode == 1) a.v_first[(size_t)t * a.ldvf + c] = x;
            if (a.vmix_mode == 2) x = (1.0f - lam) * x + lam * a.v_first[(size_t)t * a.ldvf + c];
            if (f32)
                reinterpret_cast<float*>(vd)[c] = x;
            else
                reinterpret_cast<uint16_t*>(vd)[c] = float_to_h16(x, bf);
        }
    }
    (void)vn;
}

// ------------------------------------------------------------------ attention over the cached rows
constexpr int kSinkWarps = 4;

// One block per (token, head, share).  Its warps take the share's 32-key chunks in turn, each with its own running
// (m, l, acc); they meet in shared memory in warp order.  The sink enters once, as the start value (m = 0, l = sink) of
// warp 0 of share 0.  splits > 1: the block leaves (acc, m, l) in part[t][h][share][vdim + 2].
template <int NPER>
__global__ void __launch_bounds__(kSinkWarps * 32) sink_attn_kernel(b200_sink_attn_args a, int splits, float* __restrict__ part) {
    extern __shared__ float sm[];                  // q [dim] | per warp: acc [vdim], m, l
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int t = blockIdx.x, h = blockIdx.y, z = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = h / (a.heads / a.kv_heads);
    const int D = a.dim, V = a.vdim;
    float* qs = sm;
    float* ws = sm + D;
    const int p = a.pos ? a.pos[t] : a.pos0 + t;
    int lo = 0, hi = p;
    if (splits > 1) {
        const int per = ((p + splits) / splits + 31) / 32 * 32;
        lo = z * per;
        hi = lo + per - 1 < p ? lo + per - 1 : p;
    }
    const float* q = a.proj + (size_t)t * a.ldp + a.q_off + (size_t)h * D;
    for (int d = tid; d < D; d += kSinkWarps * 32) qs[d] = q[d];
    __syncthreads();
    const bool f32 = a.cache_dtype == B200_F32;
    const int bf = a.cache_dtype == B200_BF16;
    const char* kb = sink_plane(a, t, 0);
    const char* vb = sink_plane(a, t, 1);
    const size_t re = (size_t)a.row_elems;
    const bool vec16 = !f32 && D % 8 == 0 && a.row_elems % 8 == 0 && (reinterpret_cast<uintptr_t>(kb) & 15) == 0;
    // value columns of a lane: lane + 32 i, or (16-bit caches, even sizes) the pairs 64 i + 2 lane, + 1
    const bool pair = !f32 && NPER % 2 == 0 && V % 2 == 0 && a.row_elems % 2 == 0 && (reinterpret_cast<uintptr_t>(vb) & 3) == 0;
    // ... or (sizes and addresses that allow 16-byte loads) 8 lanes per key with 8 neighbouring columns each, four keys
    // per pass: the lanes of a subgroup sum over their keys, the subgroups meet at the end
    const bool vecv = vec16 && NPER % 2 == 0 && V % 8 == 0 && (reinterpret_cast<uintptr_t>(vb) & 15) == 0;
    const bool sink_here = warp == 0 && z == 0 && a.sink > 0.f;
    float m = sink_here ? 0.f : -INFINITY, l = sink_here ? a.sink : 0.f, acc[NPER];
    float accv[NPER / 2 > 0 ? NPER / 2 : 1][8];
#pragma unroll
    for (int i = 0; i < NPER; ++i) acc[i] = 0.f;
#pragma unroll
    for (int i = 0; i < (NPER / 2 > 0 ? NPER / 2 : 1); ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) accv[i][e] = 0.f;
    for (int j0 = lo + warp * 32; j0 <= hi; j0 += kSinkWarps * 32) {
        const int n = hi - j0 + 1 < 32 ? hi - j0 + 1 : 32;
        float s = -INFINITY;
        if (vec16) {
            // 8 lanes share a key (128 contiguous bytes per pass), 4 keys per instruction; lane L ends up with the score
            // of key L, which pass L / 4 computed in subgroup L % 4
            const int part = lane & 7, sg = lane >> 3;
            const uint16_t* kbase = reinterpret_cast<const uint16_t*>(kb) + (size_t)g * D;
#pragma unroll
            for (int it = 0; it < 8; ++it) {          // (unrolled: the passes' loads are all in flight together)
                const int jj = it * 4 + sg < n ? it * 4 + sg : n - 1;     // (beyond the chunk: a valid row, result unused)
                float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
                {
                    const uint16_t* kr = kbase + (size_t)(j0 + jj) * re;
                    for (int c = part * 8; c < D; c += 64) {
                        const uint4 v = *reinterpret_cast<const uint4*>(kr + c);
                        const float4 qa = *reinterpret_cast<const float4*>(qs + c), qb = *reinterpret_cast<const float4*>(qs + c + 4);
                        d0 = fmaf(qa.x, h16_to_float((uint16_t)(v.x & 0xffff), bf), d0);
                        d1 = fmaf(qa.y, h16_to_float((uint16_t)(v.x >> 16), bf), d1);
                        d2 = fmaf(qa.z, h16_to_float((uint16_t)(v.y & 0xffff), bf), d2);
                        d3 = fmaf(qa.w, h16_to_float((uint16_t)(v.y >> 16), bf), d3);
                        d0 = fmaf(qb.x, h16_to_float((uint16_t)(v.z & 0xffff), bf), d0);
                        d1 = fmaf(qb.y, h16_to_float((uint16_t)(v.z >> 16), bf), d1);
                        d2 = fmaf(qb.z, h16_to_float((uint16_t)(v.w & 0xffff), bf), d2);
                        d3 = fmaf(qb.w, h16_to_float((uint16_t)(v.w >> 16), bf), d3);
                    }
                }
                float d = (d0 + d1) + (d2 + d3);
                d += __shfl_xor_sync(0xffffffffu, d, 1);
                d += __shfl_xor_sync(0xffffffffu, d, 2);
                d += __shfl_xor_sync(0xffffffffu, d, 4);
                const float got = __shfl_sync(0xffffffffu, d, (lane & 3) * 8);
                if ((lane >> 2) == it) s = got;
            }
            if (lane >= n) s = -INFINITY;
        } else if (lane < n) {
            float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
            {
                const size_t base = (size_t)(j0 + lane) * re + (size_t)g * D;
                int d = 0;
                for (; d + 4 <= D; d += 4) {
                    float k0, k1, k2, k3;
                    if (f32) {
                        const float* kr = reinterpret_cast<const float*>(kb) + base + d;
                        k0 = kr[0], k1 = kr[1], k2 = kr[2], k3 = kr[3];
                    } else {
                        const uint16_t* kr = reinterpret_cast<const uint16_t*>(kb) + base + d;
                        k0 = h16_to_float(kr[0], bf), k1 = h16_to_float(kr[1], bf), k2 = h16_to_float(kr[2], bf), k3 = h16_to_float(kr[3], bf);
                    }
                    d0 = fmaf(qs[d], k0, d0);
                    d1 = fmaf(qs[d + 1], k1, d1);
                    d2 = fmaf(qs[d + 2], k2, d2);
                    d3 = fmaf(qs[d + 3], k3, d3);
                }
                for (; d < D; ++d)
                    d0 = fmaf(qs[d], f32 ? reinterpret_cast<const float*>(kb)[base + d]
                                         : h16_to_float(reinterpret_cast<const uint16_t*>(kb)[base + d], bf), d0);
            }
            s = (d0 + d1) + (d2 + d3);
        }
        float cm = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
        const float mn = fmaxf(m, cm);                       // finite: the chunk holds at least one key
        const float alpha = expf(m - mn);                    // first chunk without a sink: exp(-inf) = 0
        const float pj = lane < n ? expf(s - mn) : 0.f;
        float ps = pj;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        l = l * alpha + ps;
        m = mn;
#pragma unroll
        for (int i = 0; i < NPER; ++i) acc[i] *= alpha;
        if (vecv) {
            const int part = lane & 7, sg = lane >> 3;
            const uint16_t* vbase = reinterpret_cast<const uint16_t*>(vb) + (size_t)g * V + part * 8;
#pragma unroll
            for (int i = 0; i < NPER / 2; ++i)
#pragma unroll
                for (int e = 0; e < 8; ++e) accv[i][e] *= alpha;
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int jj = it * 4 + sg, jc = jj < n ? jj : n - 1;
                const float wj = __shfl_sync(0xffffffffu, pj, jc);
                const float w = jj < n ? wj : 0.f;
#pragma unroll
                for (int i = 0; i < NPER / 2; ++i) {
                    if (64 * i + part * 8 < V) {
                        const uint4 x = *reinterpret_cast<const uint4*>(vbase + (size_t)(j0 + jc) * re + 64 * i);
                        accv[i][0] = fmaf(w, h16_to_float((uint16_t)(x.x & 0xffff), bf), accv[i][0]);
                        accv[i][1] = fmaf(w, h16_to_float((uint16_t)(x.x >> 16), bf), accv[i][1]);
                        accv[i][2] = fmaf(w, h16_to_float((uint16_t)(x.y & 0xffff), bf), accv[i][2]);
                        accv[i][3] = fmaf(w, h16_to_float((uint16_t)(x.y >> 16), bf), accv[i][3]);
                        accv[i][4] = fmaf(w, h16_to_float((uint16_t)(x.z & 0xffff), bf), accv[i][4]);
                        accv[i][5] = fmaf(w, h16_to_float((uint16_t)(x.z >> 16), bf), accv[i][5]);
                        accv[i][6] = fmaf(w, h16_to_float((uint16_t)(x.w & 0xffff), bf), accv[i][6]);
                        accv[i][7] = fmaf(w, h16_to_float((uint16_t)(x.w >> 16), bf), accv[i][7]);
                    }
                }
            }
        } else if (pair) {   // two neighbouring 16-bit values per lane and load: 128 contiguous bytes per warp
            const uint16_t* vrow = reinterpret_cast<const uint16_t*>(vb) + (size_t)j0 * re + (size_t)g * V + 2 * lane;
#pragma unroll 8
            for (int j = 0; j < n; ++j) {
                const float w = __shfl_sync(0xffffffffu, pj, j);
#pragma unroll
                for (int i = 0; i < NPER / 2; ++i) {
                    if (64 * i + 2 * lane < V) {
                        const uint32_t x = *reinterpret_cast<const uint32_t*>(vrow + (size_t)j * re + 64 * i);
                        acc[2 * i] = fmaf(w, h16_to_float((uint16_t)(x & 0xffff), bf), acc[2 * i]);
                        acc[2 * i + 1] = fmaf(w, h16_to_float((uint16_t)(x >> 16), bf), acc[2 * i + 1]);
                    }
                }
            }
        } else {
            for (int j = 0; j < n; ++j) {
                const float w = __shfl_sync(0xffffffffu, pj, j);
                const size_t base = (size_t)(j0 + j) * re + (size_t)g * V;
#pragma unroll
                for (int i = 0; i < NPER; ++i) {
                    const int d = lane + 32 * i;
                    if (d < V) {
                        const float v = f32 ? reinterpret_cast<const float*>(vb)[base + d]
                                            : h16_to_float(reinterpret_cast<const uint16_t*>(vb)[base + d], bf);
                        acc[i] = fmaf(w, v, acc[i]);
                    }
                }
            }
        }
    }
    // the warps' shares meet in warp order
    float* mine = ws + warp * (V + 2);
    if (vecv) {
#pragma unroll
        for (int i = 0; i < NPER / 2; ++i) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                float v = accv[i][e];
                v += __shfl_xor_sync(0xffffffffu, v, 8);
                v += __shfl_xor_sync(0xffffffffu, v, 16);
                const int d = 64 * i + (lane & 7) * 8 + e;
                if (lane < 8 && d < V) mine[d] = v;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < NPER; ++i) {
            const int d = pair ? 64 * (i / 2) + 2 * lane + (i & 1) : lane + 32 * i;
            if (d < V) mine[d] = acc[i];
        }
    }
    if (lane == 0) {
        mine[V] = m;
        mine[V + 1] = l;
    }
    __syncthreads();
    if (warp != 0) return;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kSinkWarps; ++w) M = fmaxf(M, ws[w * (V + 2) + V]);
    float L = 0.f, wgt[kSinkWarps];
#pragma unroll
    for (int w = 0; w < kSinkWarps; ++w) {
        const float mw = ws[w * (V + 2) + V];
        wgt[w] = mw > -INFINITY ? expf(mw - M) : 0.f;
        L += ws[w * (V + 2) + V + 1] * wgt[w];
    }
    float* po = splits > 1 ? part + (((size_t)t * a.heads + h) * splits + z) * (V + 2) : nullptr;
    const float gate = 1.0f / (1.0f + expf(-a.proj[(size_t)t * a.ldp + a.g_off + h]));
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
        const int d = lane + 32 * i;
        if (d >= V) continue;
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < kSinkWarps; ++w) o += wgt[w] * ws[w * (V + 2) + d];
        if (po) {
            po[d] = o;
        } else {
            const float y = o / L * gate;
            const size_t at = (size_t)t * a.ldo + (size_t)h * V + d;
            if (a.out_dtype == B200_F32)
                static_cast<float*>(a.out)[at] = y;
            else
                static_cast<uint16_t*>(a.out)[at] = float_to_h16(y, a.out_dtype == B200_BF16);
        }
    }
    if (po && lane == 0) {                                   // (a share without keys or sink leaves m = -inf, l = 0)
        po[V] = M;
        po[V + 1] = L;
    }
}

// One warp per (token, head, 32 output columns): the shares' (acc, m, l) merged in index order, normalised and gated.
__global__ void __launch_bounds__(128) sink_merge_kernel(b200_sink_attn_args a, const float* __restrict__ part, int splits) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int V = a.vdim, slices = (V + 31) / 32;
    const int w = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= a.T * a.heads * slices) return;
    const int th = w / slices, d = (w - th * slices) * 32 + lane;
    const int t = th / a.heads, h = th - t * a.heads;
    const float* p = part + (size_t)th * splits * (V + 2);
    const float ms = lane < splits ? p[(size_t)lane * (V + 2) + V] : -INFINITY;
    const float ls = lane < splits ? p[(size_t)lane * (V + 2) + V + 1] : 0.f;
    float m = ms;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float wsh = ms > -INFINITY ? expf(ms - m) : 0.f;
    float l = 0.f, acc = 0.f;
    for (int s = 0; s < splits; ++s) {
        const float wv = __shfl_sync(0xffffffffu, wsh, s);
        l += __shfl_sync(0xffffffffu, ls, s) * wv;
        if (d < V && wv != 0.f) acc += wv * p[(size_t)s * (V + 2) + d];
    }
    if (d >= V) return;
    const float gate = 1.0f / (1.0f + expf(-a.proj[(size_t)t * a.ldp + a.g_off + h]));
    const float y = acc / l * gate;
    const size_t at = (size_t)t * a.ldo + (size_t)h * V + d;
    if (a.out_dtype == B200_F32)
        static_cast<float*>(a.out)[at] = y;
    else
        static_cast<uint16_t*>(a.out)[at] = float_to_h16(y, a.out_dtype == B200_BF16);
}

template <int NPER>
static int launch_sink_attn(const b200_sink_attn_args* a, cudaStream_t s, int splits, float* part) {
    const size_t smem = ((size_t)a->dim + (size_t)kSinkWarps * (a->vdim + 2)) * sizeof(float);
    dim3 grid(a->T, a->heads, splits);
    B200_CUDA_CHECK(launch(sink_attn_kernel<NPER>, grid, dim3(kSinkWarps * 32), smem, s, a->pdl != 0, *a, splits, part));
    if (splits > 1)
        B200_CUDA_CHECK(launch(sink_merge_kernel, dim3((a->T * a->heads * ((a->vdim + 31) / 32) + 3) / 4), dim3(128), 0, s,
                               a->pdl != 0, *a, (const float*)part, splits));
    return B200_OK;
}

}  // namespace b200

using namespace b200;

static int check_sink(const b200_sink_attn_args* a, const char* who) {
    if (!a || !a->proj || ((!a->k_cache || !a->v_cache) && !a->kv_ptrs)) return fail(B200_EINVAL, "%s: null pointer argument", who);
    if (a->T <= 0 || a->heads <= 0 || a->kv_heads <= 0 || a->heads % a->kv_heads || a->dim <= 0 || a->vdim <= 0 ||
        a->row_elems < a->kv_heads * a->dim || a->row_elems < a->kv_heads * a->vdim)
        return fail(B200_EINVAL, "%s: bad sizes (heads %d kv_heads %d dim %d vdim %d row %d)", who, a->heads, a->kv_heads, a->dim,
                    a->vdim, a->row_elems);
    if (a->cache_dtype != B200_F32 && a->cache_dtype != B200_BF16 && a->cache_dtype != B200_F16)
        return fail(B200_EINVAL, "%s: bad cache element type %d", who, a->cache_dtype);
    return B200_OK;
}

extern "C" int b200_sink_attn_append(const b200_sink_attn_args* a, void* stream) {
    if (int rc = check_sink(a, "b200_sink_attn_append")) return rc;
    if (!a->q_gain || !a->k_gain) return fail(B200_EINVAL, "b200_sink_attn_append: norm gains missing");
    if (a->vmix_mode < 0 || a->vmix_mode > 2 || (a->vmix_mode && !a->v_first) || (a->vmix_mode == 2 && !a->vmix))
        return fail(B200_EINVAL, "b200_sink_attn_append: value blending without its operands");
    B200_CUDA_CHECK(launch(sink_attn_append_kernel, dim3(a->T, 3), dim3(256), 0, static_cast<cudaStream_t>(stream), a->pdl != 0, *a));
    return B200_OK;
}

extern "C" int64_t b200_sink_attn_scratch_bytes(int32_t T, int32_t heads, int32_t vdim, int32_t splits) {
    return (int64_t)T * heads * splits * (vdim + 2) * (int64_t)sizeof(float);
}

extern "C" int b200_sink_attn(const b200_sink_attn_args* a, int32_t splits, float* scratch, void* stream) {
    if (int rc = check_sink(a, "b200_sink_attn")) return rc;
    if (!a->out) return fail(B200_EINVAL, "b200_sink_attn: out missing");
    if (splits < 1 || splits > 32 || (splits > 1 && !scratch)) return fail(B200_EINVAL, "b200_sink_attn: bad splits %d", splits);
    if (a->dim + kSinkWarps * (a->vdim + 2) > 11 * 1024) return fail(B200_ELIMIT, "b200_sink_attn: dim %d / vdim %d too large", a->dim, a->vdim);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int nper = (a->vdim + 31) / 32;
    if (nper <= 1) return launch_sink_attn<1>(a, s, splits, scratch);
    if (nper <= 2) return launch_sink_attn<2>(a, s, splits, scratch);
    if (nper <= 4) return launch_sink_attn<4>(a, s, splits, scratch);
    if (nper <= 8) return launch_sink_attn<8>(a, s, splits, scratch);
    if (nper <= 16) return launch_sink_attn<16>(a, s, splits, scratch);
    return fail(B200_ELIMIT, "b200_sink_attn: vdim %d > 512", a->vdim);
}
