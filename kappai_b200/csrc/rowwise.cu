// Row-wise kernels: embedding gather, RMSNorm, SwiGLU, casts.
// One row's result never depends on the other rows of the launch.
#include "common.cuh"

// x[r,:] = float(table[ids[r],:])            (src/backend/cpu/common.c:1774-1782)
// `scale` multiplies the row (1.0 = none; the architecture decides).  With a table of learned position vectors
// (`pos_table`, rows by position) the row of the token's position is added, unscaled.
template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                  float* __restrict__ x, int d, float scale, const T* __restrict__ pos_table,
                                  const int* __restrict__ positions) {
    kp_pdl_begin();
    const int r = blockIdx.x;
    const T* src = table + (size_t)ids[r] * d;
    float* dst = x + (size_t)r * d;
    if (pos_table != nullptr) {
        const T* ps = pos_table + (size_t)positions[r] * d;
        for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = fmaf(to_f32(src[i]), scale, to_f32(ps[i]));
        return;
    }
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = to_f32(src[i]) * scale;
}

// y[r,:] = (x[row,:] * rsqrt(mean(x^2) + eps)) * w     (src/backend/cpu/scalar/quants.c:1489-1512)
// row = rows ? rows[r] : r.  The sum of squares is float32 with a fixed tree.
template <typename T>
__global__ void rmsnorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                    T* __restrict__ y, const int* __restrict__ rows, int d, float eps) {
    kp_pdl_begin();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float* src = x + (size_t)(rows ? rows[r] : r) * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = src[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    T* dst = y + (size_t)r * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = from_f32<T>((src[i] * scale) * w[i]);
}

// four consecutive outputs in one store (the destination is 8- or 16-byte aligned: d % 4 == 0)
__device__ __forceinline__ void store4(float* dst, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(bf16* dst, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = o;
}

// The same for rows of at most 8192 floats that are 16-byte aligned: each thread keeps its 8 float4 of the
// row in registers, so the row is read once.
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_rows_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ y,
                        const int* __restrict__ rows, int d, float eps) {
    kp_pdl_begin();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * d);
    const int n4 = d >> 2;
    float4 v[8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int i = threadIdx.x + j * 256;
        v[j] = i < n4 ? __ldg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
        ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
        ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    T* dst = y + (size_t)r * d;
    const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int i = threadIdx.x + j * 256;
        if (i < n4) {
            const float4 ww = __ldg(w4 + i);
            store4(dst + 4 * i, (v[j].x * scale) * ww.x, (v[j].y * scale) * ww.y, (v[j].z * scale) * ww.z,
                   (v[j].w * scale) * ww.w);
        }
    }
}

// Rows of at most 2048 elements (a multiple of 4), two kernels with ONE arithmetic, so that which of them runs
// (it depends on the number of rows) changes no bit of the result.  The row is 16 groups of 32 float4; "lane" l
// of "part" g (0..7) sums the squares of float4 l of group g, then of group g + 8, in element order; a lane's
// eight parts are added in order of g; the 32 lane sums are added by the warp butterfly.
//  * warp kernel (many rows): one warp a row, the row in registers (all loads in flight at once), no
//    block-wide barrier, eight rows a block.
//  * block kernel (few rows): 256 threads a row (thread = (part, lane)), so that a row's loads are spread
//    over more threads and the rows over more SMs.
__device__ __forceinline__ float sumsq8(const float4& a, const float4& b) {
    float ss = 0.f;
    ss = fmaf(a.x, a.x, ss); ss = fmaf(a.y, a.y, ss); ss = fmaf(a.z, a.z, ss); ss = fmaf(a.w, a.w, ss);
    ss = fmaf(b.x, b.x, ss); ss = fmaf(b.y, b.y, ss); ss = fmaf(b.z, b.z, ss); ss = fmaf(b.w, b.w, ss);
    return ss;
}

template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_rows_warp_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ y,
                         const int* __restrict__ rows, int n, int d, float eps) {
    kp_pdl_begin();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= n) return;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * d);
    const int n4 = d >> 2;
    float4 v[16];
#pragma unroll
    for (int j = 0; j < 16; j++) {
        const int i = lane + j * 32;
        v[j] = i < n4 ? __ldg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float ss = sumsq8(v[0], v[8]);
#pragma unroll
    for (int g = 1; g < 8; g++) ss += sumsq8(v[g], v[g + 8]);
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    T* dst = y + (size_t)r * d;
    const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll
    for (int j = 0; j < 16; j++) {
        const int i = lane + j * 32;
        if (i < n4) {
            const float4 ww = __ldg(w4 + i);
            store4(dst + 4 * i, (v[j].x * scale) * ww.x, (v[j].y * scale) * ww.y, (v[j].z * scale) * ww.z,
                   (v[j].w * scale) * ww.w);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_rows_blk_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ y,
                        const int* __restrict__ rows, int d, float eps) {
    kp_pdl_begin_early();       // (measured with one row as well: a decode step 609 -> 601 us)
    __shared__ float part[8][32];
    __shared__ float scale_s;
    const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
    const int r = blockIdx.x;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * d);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    const int n4 = d >> 2;
    const int ia = lane + 32 * g, ib = lane + 32 * (g + 8);
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 a = ia < n4 ? __ldg(src + ia) : zero, b = ib < n4 ? __ldg(src + ib) : zero;
    const float4 wa = ia < n4 ? __ldg(w4 + ia) : zero, wb = ib < n4 ? __ldg(w4 + ib) : zero;
    part[g][lane] = sumsq8(a, b);
    __syncthreads();
    if (g == 0) {
        float ss = part[0][lane];
#pragma unroll
        for (int k = 1; k < 8; k++) ss += part[k][lane];
        ss = warp_sum(ss);
        if (lane == 0) scale_s = 1.0f / sqrtf(ss / (float)d + eps);
    }
    __syncthreads();
    const float scale = scale_s;
    T* dst = y + (size_t)r * d;
    if (ia < n4) store4(dst + 4 * ia, (a.x * scale) * wa.x, (a.y * scale) * wa.y, (a.z * scale) * wa.z, (a.w * scale) * wa.w);
    if (ib < n4) store4(dst + 4 * ib, (b.x * scale) * wb.x, (b.y * scale) * wb.y, (b.z * scale) * wb.z, (b.w * scale) * wb.w);
}

// Post-norm step of a residual layer: y = (a * rsqrt(mean(a^2) + eps)) * w for the rows a of `acc` (the
// float32 sum alpha * x + sublayer(x) of a layer that norms AFTER the sum).  Up to three images of y leave in
// one pass, each only if its pointer is given: y itself in float32 (`x_out`, the new residual), y in the
// storage type (`h_out`, what the next sublayer's products read) and alpha * y in float32 (`scaled_out`, the
// sum the next sublayer adds into).  Every output may be `acc` itself: an element is read and written by the
// same thread, after the row's statistic is known.
template <typename T>
__global__ void __launch_bounds__(256)
postnorm_rows_kernel(const float* acc, const float* __restrict__ w, float* x_out, T* h_out, float* scaled_out,
                     int d, float eps, float alpha) {
    kp_pdl_begin();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float* src = acc + (size_t)r * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = src[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float y = (src[i] * scale) * w[i];
        if (x_out) x_out[(size_t)r * d + i] = y;
        if (h_out) h_out[(size_t)r * d + i] = from_f32<T>(y);
        if (scaled_out) scaled_out[(size_t)r * d + i] = alpha * y;
    }
}

// The same for 16-byte aligned rows of at most 8192 floats (d % 4 == 0): a thread keeps its float4s of the row in
// registers, so the row is read once and leaves in 16- and 8-byte stores.
template <typename T>
__global__ void __launch_bounds__(256)
postnorm_rows_vec_kernel(const float* acc, const float* __restrict__ w, float* x_out, T* h_out, float* scaled_out,
                         int d, float eps, float alpha) {
    kp_pdl_begin();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float4* src = reinterpret_cast<const float4*>(acc + (size_t)r * d);
    const int n4 = d >> 2;
    float4 v[8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int i = threadIdx.x + j * 256;
        v[j] = i < n4 ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
        ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
        ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int i = threadIdx.x + j * 256;
        if (i < n4) {
            const float4 ww = __ldg(w4 + i);
            const float a = (v[j].x * scale) * ww.x, b = (v[j].y * scale) * ww.y, c = (v[j].z * scale) * ww.z,
                        e = (v[j].w * scale) * ww.w;
            const size_t o = (size_t)r * d + 4 * (size_t)i;
            if (x_out) store4(x_out + o, a, b, c, e);
            if (h_out) store4(h_out + o, a, b, c, e);
            if (scaled_out) store4(scaled_out + o, alpha * a, alpha * b, alpha * c, alpha * e);
        }
    }
}

// The entry of such a layer when nothing has prepared it: h = x in the storage type, scaled = alpha * x.
template <typename T>
__global__ void scale_cast_kernel(const float* __restrict__ x, T* __restrict__ h_out, float* __restrict__ scaled_out,
                                  size_t n, float alpha) {
    kp_pdl_begin();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = x[i];
        if (h_out) h_out[i] = from_f32<T>(v);
        scaled_out[i] = alpha * v;
    }
}

// o[r, c] *= sigmoid(g[r, c]): an output gate on the concatenated heads, the gate being columns of a wider
// row (the product that also made q and k).  The sigmoid is float32.
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ o, int ldo, const T* __restrict__ g, int ldg, int n, int cols) {
    kp_pdl_begin();
    const size_t total = (size_t)n * cols;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / cols, c = i % cols;
        const float z = to_f32(g[r * ldg + c]);
        T* p = o + r * ldo + c;
        *p = from_f32<T>(to_f32(*p) * (1.0f / (1.0f + expf(-z))));
    }
}

// The same, eight bfloat16 a thread, for 16-byte aligned rows whose length is a multiple of 8.
__global__ void sigmoid_gate_vec_kernel(bf16* __restrict__ o, int ldo, const bf16* __restrict__ g, int ldg, int n, int cols8) {
    kp_pdl_begin();
    const size_t total = (size_t)n * cols8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / cols8, c = (i % cols8) * 8;
        uint4 ov = *reinterpret_cast<const uint4*>(o + r * ldo + c);
        const uint4 gv = *reinterpret_cast<const uint4*>(g + r * ldg + c);
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 a = __bfloat1622float2(o2[j]), z = __bfloat1622float2(g2[j]);
            o2[j] = __floats2bfloat162_rn(a.x * (1.0f / (1.0f + expf(-z.x))), a.y * (1.0f / (1.0f + expf(-z.y))));
        }
        *reinterpret_cast<uint4*>(o + r * ldo + c) = ov;
    }
}

// act = f(gate) * up with f = silu, g / (1 + exp(-g))     (src/backend/cpu/scalar/core.c:774-800),
// relu or tanh-gelu (`act_kind`, see common.cuh).  gate_up rows hold [gate(ff) | up(ff)].
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ act, int n, int ff, int act_kind) {
    kp_pdl_begin();
    const size_t total = (size_t)n * ff;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / ff, c = i % ff;
        const float g = to_f32(gu[r * 2 * ff + c]);
        const float u = to_f32(gu[r * 2 * ff + ff + c]);
        act[i] = from_f32<T>(kp_act_rt(act_kind, g) * u);
    }
}


// RMS norm of one or two column stretches of rows in the storage type: out_s[r, :] = norm(in[r, c_s : c_s + w_s]) * wt_s
// (float32 statistics).  For latents that leave one product side by side and are normed each on its own.
struct ColNorm { int col, width, ld_out; const float* weight; void* out; };
template <typename T>
__global__ void __launch_bounds__(128)
rmsnorm_cols_kernel(const T* __restrict__ in, int ld, ColNorm a, ColNorm b, float eps) {
    kp_pdl_begin();
    __shared__ float red[32];
    const ColNorm c = blockIdx.y == 0 ? a : b;
    const int r = blockIdx.x;
    const T* src = in + (size_t)r * ld + c.col;
    float ss = 0.f;
    for (int i = threadIdx.x; i < c.width; i += blockDim.x) {
        const float v = to_f32(src[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)c.width + eps);
    T* dst = (T*)c.out + (size_t)r * c.ld_out;
    for (int i = threadIdx.x; i < c.width; i += blockDim.x) dst[i] = from_f32<T>((to_f32(src[i]) * scale) * c.weight[i]);
}

// out[r, :] = norm(o[r, :]) * w * sigmoid(g[r, :]): the RMS norm of float32 rows (all heads of a mixer's output
// together) and the output gate in one pass; `g` is columns of a wider row in the storage type.
template <typename T>
__global__ void __launch_bounds__(256)
norm_gate_rows_kernel(const float* __restrict__ o, const float* __restrict__ w, const T* __restrict__ g, int ldg,
                      T* __restrict__ out, int ldo, int d, float eps) {
    kp_pdl_begin();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float* src = o + (size_t)r * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = src[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float z = to_f32(g[(size_t)r * ldg + i]);
        out[(size_t)r * ldo + i] = from_f32<T>(((src[i] * scale) * w[i]) * (1.0f / (1.0f + expf(-z))));
    }
}

// out[r, c] = act(gate[r, c]) * table[ids[r], col0 + c]: a gate on a stretch of a second token table's row.
template <typename T>
__global__ void token_gate_kernel(const T* __restrict__ gate, int ldg, const T* __restrict__ table, int ldt, int col0,
                                  const int* __restrict__ ids, T* __restrict__ out, int n, int dim, int act_kind) {
    kp_pdl_begin();
    const size_t total = (size_t)n * dim;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / dim, c = i % dim;
        const float z = to_f32(gate[r * ldg + c]);
        const float e = to_f32(table[(size_t)ids[r] * ldt + col0 + c]);
        out[i] = from_f32<T>(kp_act_rt(act_kind, z) * e);
    }
}

// x[r, :] += norm(y[r, :]) * w for float32 rows: a branch that is normed before it joins the residual.
__global__ void __launch_bounds__(256)
rmsnorm_add_rows_kernel(const float* __restrict__ y, const float* __restrict__ w, float* __restrict__ x, int d, float eps) {
    kp_pdl_begin();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float* src = y + (size_t)r * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = src[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) x[(size_t)r * d + i] += (src[i] * scale) * w[i];
}

// A branch that is normed before it joins the residual, for layers that norm a sublayer on both sides:
//   x[r, :] += norm(y[r, :]) * wb ;  y[r, :] = 0 ;  and, if h_out is given, h_out[r, :] = norm(x[r, :]) * wn
// (the new x; h_out in the storage type: what the sublayer after this one reads).  All statistics float32 with a
// fixed tree; the branch is cleared for whoever adds into it next.  Rows of at most 256 * RMS_ADD_KEEP floats stay
// in registers between the passes, longer ones are read again.
#define RMS_ADD_KEEP 16
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_add_norm_rows_kernel(float* __restrict__ y, const float* __restrict__ wb, float eps_b, float* __restrict__ x,
                             const float* __restrict__ wn, float eps_n, T* __restrict__ h_out, int d) {
    kp_pdl_begin();
    __shared__ float red[32];
    const int r = blockIdx.x;
    float* yr = y + (size_t)r * d;
    float* xr = x + (size_t)r * d;
    const bool keep = d <= 256 * RMS_ADD_KEEP;
    float v[RMS_ADD_KEEP];
    float ss = 0.f;
    if (keep) {
#pragma unroll
        for (int j = 0; j < RMS_ADD_KEEP; j++) {
            const int i = threadIdx.x + j * 256;
            v[j] = i < d ? yr[i] : 0.f;
            ss = fmaf(v[j], v[j], ss);
        }
    } else {
        for (int i = threadIdx.x; i < d; i += 256) { const float a = yr[i]; ss = fmaf(a, a, ss); }
    }
    ss = block_sum(ss, red);
    const float sb = 1.0f / sqrtf(ss / (float)d + eps_b);
    float s2 = 0.f;
    if (keep) {
#pragma unroll
        for (int j = 0; j < RMS_ADD_KEEP; j++) {
            const int i = threadIdx.x + j * 256;
            if (i < d) {
                v[j] = xr[i] + (v[j] * sb) * wb[i];
                xr[i] = v[j];
                yr[i] = 0.f;
                s2 = fmaf(v[j], v[j], s2);
            }
        }
    } else {
        for (int i = threadIdx.x; i < d; i += 256) {
            const float a = xr[i] + (yr[i] * sb) * wb[i];
            xr[i] = a;
            yr[i] = 0.f;
            s2 = fmaf(a, a, s2);
        }
    }
    if (h_out == nullptr) return;
    s2 = block_sum(s2, red);
    const float sn = 1.0f / sqrtf(s2 / (float)d + eps_n);
    T* hr = h_out + (size_t)r * d;
    if (keep) {
#pragma unroll
        for (int j = 0; j < RMS_ADD_KEEP; j++) {
            const int i = threadIdx.x + j * 256;
            if (i < d) hr[i] = from_f32<T>((v[j] * sn) * wn[i]);
        }
    } else {
        for (int i = threadIdx.x; i < d; i += 256) hr[i] = from_f32<T>((xr[i] * sn) * wn[i]);
    }
}

// The same for 16-byte aligned rows of at most 8192 floats (d % 4 == 0): a thread keeps its float4s of the row in
// registers, so y and x are read once, and x, the cleared y and h leave in 16- and 8-byte stores.  Which form runs
// depends on the row's length and the buffers' alignment alone, never on the rows of the step.  PER: float4s a thread
// (2, 4 or 8 by the row's length: the fewer registers hold the row, the more rows an SM has in flight).
template <typename T, int PER>
__global__ void __launch_bounds__(256)
rmsnorm_add_norm_rows_vec_kernel(float* __restrict__ y, const float* __restrict__ wb, float eps_b, float* __restrict__ x,
                                 const float* __restrict__ wn, float eps_n, T* __restrict__ h_out, int d) {
    kp_pdl_begin();
    __shared__ float red[32];
    const int r = blockIdx.x, d4 = d >> 2;
    float4* yr = reinterpret_cast<float4*>(y + (size_t)r * d);
    float4* xr = reinterpret_cast<float4*>(x + (size_t)r * d);
    float4 v[PER], xv[PER];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const int i = threadIdx.x + j * 256;
        v[j] = i < d4 ? yr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < d4) xv[j] = xr[i];
        ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss); ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
    }
    ss = block_sum(ss, red);
    const float sb = 1.0f / sqrtf(ss / (float)d + eps_b);
    float s2 = 0.f;
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const int i = threadIdx.x + j * 256;
        if (i < d4) {
            const float4 w = __ldg(reinterpret_cast<const float4*>(wb) + i);
            float4 a;
            a.x = xv[j].x + (v[j].x * sb) * w.x; a.y = xv[j].y + (v[j].y * sb) * w.y;
            a.z = xv[j].z + (v[j].z * sb) * w.z; a.w = xv[j].w + (v[j].w * sb) * w.w;
            xr[i] = a;
            yr[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            v[j] = a;
            s2 = fmaf(a.x, a.x, s2); s2 = fmaf(a.y, a.y, s2); s2 = fmaf(a.z, a.z, s2); s2 = fmaf(a.w, a.w, s2);
        }
    }
    if (h_out == nullptr) return;
    s2 = block_sum(s2, red);
    const float sn = 1.0f / sqrtf(s2 / (float)d + eps_n);
    T* hr = h_out + (size_t)r * d;
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const int i = threadIdx.x + j * 256;
        if (i < d4) {
            const float4 w = __ldg(reinterpret_cast<const float4*>(wn) + i);
            store4(hr + 4 * i, (v[j].x * sn) * w.x, (v[j].y * sn) * w.y, (v[j].z * sn) * w.z, (v[j].w * sn) * w.w);
        }
    }
}

// out[r, :] += sigmoid(h[r, :] . wg) * y[r, :]: a branch weighed by one gate a row, the gate's logit computed here
// (float32 sum in a fixed order, h widened from its storage type).
template <typename T>
__global__ void __launch_bounds__(256)
row_gate_add_kernel(const T* __restrict__ h, int ldh, const float* __restrict__ wg, const float* __restrict__ y,
                    float* __restrict__ out, int d) {
    kp_pdl_begin();
    __shared__ float red[32];
    const int r = blockIdx.x;
    float s = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) s = fmaf(to_f32(h[(size_t)r * ldh + i]), wg[i], s);
    s = block_sum(s, red);
    const float gate = 1.0f / (1.0f + expf(-s));
    for (int i = threadIdx.x; i < d; i += blockDim.x) out[(size_t)r * d + i] = fmaf(gate, y[(size_t)r * d + i], out[(size_t)r * d + i]);
}

template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n) {
    kp_pdl_begin();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(to_f32(in[i]));
}

// A weighted layer norm without a shift: y[r,:] = (x[row,:] - mean) / sqrt(var + eps) * w, var the mean of the squared
// deviations (taken about the mean, in a second pass over the row, not as a difference of two sums).  row = rows ?
// rows[r] : r.  float32 statistics with a fixed tree.
template <typename T>
__global__ void __launch_bounds__(256)
layernorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ y,
                      const int* __restrict__ rows, int d, float eps) {
    kp_pdl_begin();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float* src = x + (size_t)(rows ? rows[r] : r) * d;
    float s = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) s += src[i];
    const float mean = block_sum(s, red) / (float)d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = src[i] - mean;
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    T* dst = y + (size_t)r * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = from_f32<T>(((src[i] - mean) * scale) * w[i]);
}

// The same for rows of at most 8192 floats (a multiple of 4) that are 16-byte aligned: each thread keeps its 8 float4
// of the row in registers, so the row is read once; mean first, then the squared deviations about it.
template <typename T>
__global__ void __launch_bounds__(256)
layernorm_rows_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ y,
                          const int* __restrict__ rows, int d, float eps) {
    kp_pdl_begin();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * d);
    const int n4 = d >> 2;
    float4 v[8];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int i = threadIdx.x + j * 256;
        v[j] = i < n4 ? __ldg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
    }
    const float mean = block_sum(s, red) / (float)d;
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int i = threadIdx.x + j * 256;
        if (i < n4) {
            v[j].x -= mean; v[j].y -= mean; v[j].z -= mean; v[j].w -= mean;
            ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
            ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
        }
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    T* dst = y + (size_t)r * d;
    const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int i = threadIdx.x + j * 256;
        if (i < n4) {
            const float4 ww = __ldg(w4 + i);
            store4(dst + 4 * i, (v[j].x * scale) * ww.x, (v[j].y * scale) * ww.y, (v[j].z * scale) * ww.z,
                   (v[j].w * scale) * ww.w);
        }
    }
}

// RMS norm of float32 rows cut into `groups` stretches of equal width, every stretch with a mean square of its own,
// and a gate from rows in the storage type: gate_first ? norm(o * act(g)) * w : norm(o) * w * act(g); w may be null (no weight); act is silu
// (gate_act 0) or the sigmoid (1).  A block takes one (row, part); its size depends on the part's width alone.
template <typename T>
__global__ void __launch_bounds__(256)
group_norm_gate_rows_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ w, const T* __restrict__ g, int ldg,
                            T* __restrict__ out, int ldout, int width, float eps, int gate_first, int gate_act) {
    kp_pdl_begin();
    __shared__ float red[32];
    const int r = blockIdx.x, c0 = blockIdx.y * width;
    const float* src = o + (size_t)r * ldo + c0;
    const T* gr = g + (size_t)r * ldg + c0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = src[i];
        if (gate_first) {
            const float z = to_f32(gr[i]);
            const float sg = 1.0f / (1.0f + expf(-z));
            v *= gate_act == 0 ? z * sg : sg;
        }
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float z = to_f32(gr[i]);
        const float sg = 1.0f / (1.0f + expf(-z));
        const float gate = gate_act == 0 ? z * sg : sg;
        float v = gate_first ? (src[i] * gate) * scale : src[i] * scale;
        if (w) v *= w[c0 + i];
        if (!gate_first) v *= gate;
        out[(size_t)r * ldout + c0 + i] = from_f32<T>(v);
    }
}

__device__ __forceinline__ float4 load4(const float* src) { return *reinterpret_cast<const float4*>(src); }
__device__ __forceinline__ float4 load4(const bf16* src) {
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    const float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(hi);
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float gn_gate(float z, int gate_act) {
    const float sg = 1.0f / (1.0f + expf(-z));
    return gate_act == 0 ? z * sg : sg;
}

// The same where a part is a multiple of 4 wide, at most 16 TEAM columns, and rows and parts start on 16 bytes (8 in
// bfloat16): TEAM threads (a warp, or the block) take one (row, part) and keep it and its gates in registers, so both
// are read once and every gate's exponential is taken once.  Which form runs depends on the part's width alone.
template <typename T, int TEAM>
__global__ void __launch_bounds__(256)
group_norm_gate_rows_vec_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ w, const T* __restrict__ g, int ldg,
                                T* __restrict__ out, int ldout, int n_items, int groups, int width, float eps, int gate_first,
                                int gate_act) {
    kp_pdl_begin();
    __shared__ float red[32];
    const int team = threadIdx.x / TEAM, lane = threadIdx.x % TEAM;
    const int item = blockIdx.x * (256 / TEAM) + team;
    const bool live = item < n_items;                      // (a whole team at once; with TEAM == 256 always true)
    const int r = live ? item / groups : 0, c0 = live ? (item % groups) * width : 0;
    const float* src = o + (size_t)r * ldo + c0;
    const T* gr = g + (size_t)r * ldg + c0;
    const int n4 = width >> 2;
    float4 v[4], gt[4];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int i = lane + j * TEAM;
        v[j] = gt[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live && i < n4) {
            v[j] = load4(src + 4 * i);
            const float4 z = load4(gr + 4 * i);
            gt[j] = make_float4(gn_gate(z.x, gate_act), gn_gate(z.y, gate_act), gn_gate(z.z, gate_act), gn_gate(z.w, gate_act));
            if (gate_first) { v[j].x *= gt[j].x; v[j].y *= gt[j].y; v[j].z *= gt[j].z; v[j].w *= gt[j].w; }
            ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
            ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
        }
    }
    ss = TEAM == 32 ? warp_sum(ss) : block_sum(ss, red);
    if (!live) return;
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    T* dst = out + (size_t)r * ldout + c0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int i = lane + j * TEAM;
        if (i < n4) {
            float4 y = make_float4(v[j].x * scale, v[j].y * scale, v[j].z * scale, v[j].w * scale);
            if (w) {
                const float4 ww = load4(w + c0 + 4 * i);
                y.x *= ww.x; y.y *= ww.y; y.z *= ww.z; y.w *= ww.w;
            }
            if (!gate_first) { y.x *= gt[j].x; y.y *= gt[j].y; y.z *= gt[j].z; y.w *= gt[j].w; }
            store4(dst + 4 * i, y.x, y.y, y.z, y.w);
        }
    }
}

// o[r, h * hd + i] *= sigmoid(g[r, h]): one gate a head.
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ o, int ldo, const T* __restrict__ g, int ldg, int n, int H, int hd) {
    kp_pdl_begin();
    const size_t cols = (size_t)H * hd, total = (size_t)n * cols;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / cols, c = i % cols;
        const float z = to_f32(g[r * ldg + c / hd]);
        T* p = o + r * ldo + c;
        *p = from_f32<T>(to_f32(*p) * (1.0f / (1.0f + expf(-z))));
    }
}

// The same, four columns a thread (head sizes that are multiples of 4, rows that start on 16 bytes, 8 in bfloat16).
template <typename T>
__global__ void head_gate_vec_kernel(T* __restrict__ o, int ldo, const T* __restrict__ g, int ldg, int n, int H, int hd) {
    kp_pdl_begin();
    const size_t cols4 = (size_t)H * hd / 4, total = (size_t)n * cols4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / cols4, c = (i % cols4) * 4;
        const float z = to_f32(g[r * ldg + c / hd]);
        const float sg = 1.0f / (1.0f + expf(-z));
        T* p = o + r * ldo + c;
        const float4 v = load4(p);
        store4(p, v.x * sg, v.y * sg, v.z * sg, v.w * sg);
    }
}

// x <- cap * tanh(x / cap), in place, float32 (a soft limit on logits).
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
    kp_pdl_begin();
    const float inv = 1.0f / cap;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] * inv);
}

// The gated unit with limits: g = min(gate, limit), u = clamp(up, -limit, limit), act = g sigmoid(alpha g) (u + shift).
// gate_up rows hold [gate(ff) | up(ff)].
template <typename T>
__global__ void glu_clamped_kernel(const T* __restrict__ gu, T* __restrict__ act, int n, int ff, float limit, float alpha, float shift) {
    kp_pdl_begin();
    const size_t total = (size_t)n * ff;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / ff, c = i % ff;
        act[i] = from_f32<T>(kp_glu_clamped(to_f32(gu[r * 2 * ff + c]), to_f32(gu[r * 2 * ff + ff + c]), limit, alpha, shift));
    }
}


static inline int grid_for(size_t total, int block) {
    size_t g = (total + block - 1) / block;
    if (g > 148 * 16) g = 148 * 16;
    if (g < 1) g = 1;
    return (int)g;
}

// The tables of a captured decode step, brought to the device by a kernel instead of a copy engine: `src` is the
// step's staging buffer in pinned host memory (the device reads it over the bus), `dst` the static buffer that the
// graph's kernels read; and, in the same launch, the step's token ids from where the sampler left them.  (A
// 2 KB cudaMemcpyAsync between two graph launches costs about 10 us of stream time, this about 3.)
__global__ void step_tables_kernel(const int4* src, int4* __restrict__ dst, int n4, const int* __restrict__ tok_src,
                                   int tok_off, int n_tok) {
    kp_pdl_begin();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    // with tokens given, their place in the tables (words tok_off ..., whole int4s) is theirs alone
    const bool toks = tok_src != nullptr && i * 4 >= tok_off && i * 4 < tok_off + (n_tok + 3) / 4 * 4;
    if (i < n4 && !toks) {
        int4 v;                                   // (a volatile load: host memory, rewritten between launches)
        asm volatile("ld.volatile.global.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src + i));
        dst[i] = v;
    }
    if (toks) {
        int* d = reinterpret_cast<int*>(dst) + i * 4;
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (i * 4 + j - tok_off < n_tok) d[j] = tok_src[i * 4 + j - tok_off];
    }
}

// The status words of a step's kernels brought together: out[0] = OR of the words at the given device
// addresses.  Launched behind a step; its one word travels to the host with the step's sampled tokens, so the
// host learns without any further synchronisation whether a kernel's bounded wait gave up.
__global__ void gather_status_kernel(const unsigned long long* __restrict__ addrs, int n, int* __restrict__ out) {
    kp_pdl_begin();
    if (threadIdx.x == 0) {
        int v = 0;
        for (int i = 0; i < n; i++) v |= *reinterpret_cast<const volatile int*>(addrs[i]);
        out[0] = v;
    }
}

extern "C" {

// pos_table / positions: both given or both null.
int kp_embed_rows(const void* table, const int* ids, float* x, int n, int d, float scale, const void* pos_table,
                  const int* positions, int dtype, void* stream) {
    if (n <= 0) return 0;
    if ((pos_table == nullptr) != (positions == nullptr)) return KP_ERR_BAD_ARG;
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(embed_rows_kernel<T>, dim3(n), dim3(256), 0, (cudaStream_t)stream, (const T*)table, ids, x, d, scale,
                                               (const T*)pos_table, positions)));
    return kp_launch_status();
}

int kp_rmsnorm_rows(const float* x, const float* w, void* y, const int* rows, int n, int d, float eps, int dtype,
                    void* stream) {
    if (n <= 0) return 0;
    if ((d & 3) == 0 && d <= 8192 && (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) == 0) {
        // which kernel runs depends on the row's size and alignment only, never on the batch
        if (d <= 2048) {
            if (n <= 256) {
                KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(rmsnorm_rows_blk_kernel<T>, dim3(n), dim3(256), 0,
                                                           (cudaStream_t)stream, x, w, (T*)y, rows, d, eps)));
            } else {
                KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(rmsnorm_rows_warp_kernel<T>, dim3((n + 7) / 8), dim3(256), 0,
                                                           (cudaStream_t)stream, x, w, (T*)y, rows, n, d, eps)));
            }
            return kp_launch_status();
        }
        KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(rmsnorm_rows_vec_kernel<T>, dim3(n), dim3(256), 0, (cudaStream_t)stream, x, w, (T*)y, rows, d, eps)));
        return kp_launch_status();
    }
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(rmsnorm_rows_kernel<T>, dim3(n), dim3(256), 0, (cudaStream_t)stream, x, w, (T*)y, rows, d, eps)));
    return kp_launch_status();
}

int kp_swiglu(const void* gate_up, void* act, int n, int ff, int act_kind, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (act_kind < 0 || act_kind > KP_ACT_GELU_TANH) return KP_ERR_BAD_ARG;
    const int g = grid_for((size_t)n * ff, 256);
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(swiglu_kernel<T>, dim3(g), dim3(256), 0, (cudaStream_t)stream, (const T*)gate_up, (T*)act, n, ff, act_kind)));
    return kp_launch_status();
}

// dtype: the type of h_out.  Any of x_out, h_out, scaled_out may be null.
int kp_postnorm_rows(const float* acc, const float* w, float* x_out, void* h_out, float* scaled_out, int n, int d,
                     float eps, float alpha, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (d < 1) return KP_ERR_BAD_ARG;
    // (which kernel runs depends on the row's size and alignment only, never on the batch)
    if ((d & 3) == 0 && d <= 8192 &&
        (((uintptr_t)acc | (uintptr_t)w | (uintptr_t)x_out | (uintptr_t)h_out | (uintptr_t)scaled_out) & 15) == 0) {
        KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(postnorm_rows_vec_kernel<T>, dim3(n), dim3(256), 0, (cudaStream_t)stream, acc, w,
                                                   x_out, (T*)h_out, scaled_out, d, eps, alpha)));
        return kp_launch_status();
    }
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(postnorm_rows_kernel<T>, dim3(n), dim3(256), 0, (cudaStream_t)stream, acc, w, x_out,
                                               (T*)h_out, scaled_out, d, eps, alpha)));
    return kp_launch_status();
}

int kp_scale_cast(const float* x, void* h_out, float* scaled_out, long long n, float alpha, int dtype, void* stream) {
    if (n <= 0) return 0;
    const int g = grid_for((size_t)n, 256);
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(scale_cast_kernel<T>, dim3(g), dim3(256), 0, (cudaStream_t)stream, x, (T*)h_out,
                                               scaled_out, (size_t)n, alpha)));
    return kp_launch_status();
}

int kp_sigmoid_gate(void* o, int ldo, const void* g, int ldg, int n, int cols, int dtype, void* stream) {
    if (n <= 0 || cols <= 0) return 0;
    if (dtype == KP_DTYPE_BF16 && cols % 8 == 0 && ldo % 8 == 0 && ldg % 8 == 0 && !(((uintptr_t)o | (uintptr_t)g) & 15)) {
        kp_launch_pdl(sigmoid_gate_vec_kernel, dim3(grid_for((size_t)n * (cols / 8), 256)), dim3(256), 0, (cudaStream_t)stream,
                      (bf16*)o, ldo, (const bf16*)g, ldg, n, cols / 8);
        return kp_launch_status();
    }
    const int gr = grid_for((size_t)n * cols, 256);
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(sigmoid_gate_kernel<T>, dim3(gr), dim3(256), 0, (cudaStream_t)stream, (T*)o, ldo,
                                               (const T*)g, ldg, n, cols)));
    return kp_launch_status();
}


// One or two column stretches of `in` [n, ld] normed each on its own (width1 = 0: one stretch only).
int kp_rmsnorm_cols(const void* in, int ld, int n, float eps, int col0, int width0, const float* w0, void* out0, int ldo0,
                    int col1, int width1, const float* w1, void* out1, int ldo1, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (width0 < 1 || width1 < 0 || col0 < 0 || col1 < 0) return KP_ERR_BAD_ARG;
    const ColNorm a = {col0, width0, ldo0, w0, out0}, b = {col1, width1, ldo1, w1, out1};
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(rmsnorm_cols_kernel<T>, dim3(n, width1 > 0 ? 2 : 1), dim3(128), 0, (cudaStream_t)stream,
                                               (const T*)in, ld, a, b, eps)));
    return kp_launch_status();
}

int kp_norm_gate_rows(const float* o, const float* w, const void* g, int ldg, void* out, int ldo, int n, int d, float eps,
                      int dtype, void* stream) {
    if (n <= 0) return 0;
    if (d < 1) return KP_ERR_BAD_ARG;
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(norm_gate_rows_kernel<T>, dim3(n), dim3(256), 0, (cudaStream_t)stream, o, w,
                                               (const T*)g, ldg, (T*)out, ldo, d, eps)));
    return kp_launch_status();
}

int kp_token_gate(const void* gate, int ldg, const void* table, int ldt, int col0, const int* ids, void* out, int n, int dim,
                  int act_kind, int dtype, void* stream) {
    if (n <= 0 || dim <= 0) return 0;
    if (act_kind < 0 || act_kind > KP_ACT_GELU_TANH || col0 < 0) return KP_ERR_BAD_ARG;
    const int gr = grid_for((size_t)n * dim, 256);
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(token_gate_kernel<T>, dim3(gr), dim3(256), 0, (cudaStream_t)stream, (const T*)gate,
                                               ldg, (const T*)table, ldt, col0, ids, (T*)out, n, dim, act_kind)));
    return kp_launch_status();
}

int kp_rmsnorm_add_rows(const float* y, const float* w, float* x, int n, int d, float eps, void* stream) {
    if (n <= 0) return 0;
    if (d < 1) return KP_ERR_BAD_ARG;
    kp_launch_pdl(rmsnorm_add_rows_kernel, dim3(n), dim3(256), 0, (cudaStream_t)stream, y, w, x, d, eps);
    return kp_launch_status();
}

// wn / h_out: both given or both null.  dtype: the type of h_out.
int kp_rmsnorm_add_norm_rows(float* y, const float* wb, float eps_b, float* x, const float* wn, float eps_n, void* h_out, int n,
                             int d, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (d < 1 || ((wn == nullptr) != (h_out == nullptr))) return KP_ERR_BAD_ARG;
    const bool vec = (d & 3) == 0 && d <= 8192 && !(((uintptr_t)y | (uintptr_t)x | (uintptr_t)wb | (uintptr_t)wn | (uintptr_t)h_out) & 15);
    if (vec) {
#define RMS_ADD_VEC(PER)                                                                                                   \
        KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(rmsnorm_add_norm_rows_vec_kernel<T, PER>, dim3(n), dim3(256), 0, (cudaStream_t)stream, \
                                                   y, wb, eps_b, x, wn, eps_n, (T*)h_out, d)))
        if (d <= 2048) RMS_ADD_VEC(2);
        else if (d <= 4096) RMS_ADD_VEC(4);
        else RMS_ADD_VEC(8);
#undef RMS_ADD_VEC
        return kp_launch_status();
    }
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(rmsnorm_add_norm_rows_kernel<T>, dim3(n), dim3(256), 0, (cudaStream_t)stream, y, wb,
                                               eps_b, x, wn, eps_n, (T*)h_out, d)));
    return kp_launch_status();
}

int kp_row_gate_add(const void* h, int ldh, const float* wg, const float* y, float* out, int n, int d, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (d < 1) return KP_ERR_BAD_ARG;
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(row_gate_add_kernel<T>, dim3(n), dim3(256), 0, (cudaStream_t)stream, (const T*)h, ldh,
                                               wg, y, out, d)));
    return kp_launch_status();
}

// dtype_in/out: 0 f32, 1 bf16
int kp_cast(const void* in, void* out, long long n, int dtype_in, int dtype_out, void* stream) {
    if (n <= 0) return 0;
    const int g = grid_for((size_t)n, 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype_in == KP_DTYPE_F32 && dtype_out == KP_DTYPE_BF16)
        kp_launch_pdl(cast_kernel<float, bf16>, dim3(g), dim3(256), 0, s, (const float*)in, (bf16*)out, (size_t)n);
    else if (dtype_in == KP_DTYPE_BF16 && dtype_out == KP_DTYPE_F32)
        kp_launch_pdl(cast_kernel<bf16, float>, dim3(g), dim3(256), 0, s, (const bf16*)in, (float*)out, (size_t)n);
    else
        return KP_ERR_BAD_ARG;
    return kp_launch_status();
}

// n_words a multiple of 4, both buffers 16-byte aligned.  tok_src (may be null): n_tok token ids on the device that
// go to words tok_off ... of dst (tok_off a multiple of 4) instead of what src holds there.
int kp_step_tables(const void* src, void* dst, int n_words, const int* tok_src, int tok_off, int n_tok, void* stream) {
    if (n_words <= 0 || (n_words & 3) || (tok_off & 3) || ((uintptr_t)src & 15) || ((uintptr_t)dst & 15)) return KP_ERR_BAD_ARG;
    if (tok_src != nullptr && (tok_off < 0 || n_tok < 0 || tok_off + n_tok > n_words)) return KP_ERR_BAD_ARG;
    const int n4 = n_words / 4;
    kp_launch_pdl(step_tables_kernel, dim3((n4 + 255) / 256), dim3(256), 0, (cudaStream_t)stream, (const int4*)src, (int4*)dst,
                  n4, tok_src, tok_off, n_tok);
    return kp_launch_status();
}

int kp_gather_status(const unsigned long long* addrs, int n, int* out, void* stream) {
    if (n < 0 || !out) return KP_ERR_BAD_ARG;
    kp_launch_pdl(gather_status_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, addrs, n, out);
    return kp_launch_status();
}

int kp_layernorm_rows(const float* x, const float* w, void* y, const int* rows, int n, int d, float eps, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (d < 1) return KP_ERR_BAD_ARG;
    // rows of at most 8192 floats that start on 16 bytes: the row is read once and stays in registers
    const bool vec = (d % 4 == 0) && d <= 8192 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) && ((uintptr_t)y % 16 == 0);
    if (vec) {
        KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(layernorm_rows_vec_kernel<T>, dim3(n), dim3(256), 0, (cudaStream_t)stream, x, w, (T*)y, rows, d, eps)));
    } else {
        KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(layernorm_rows_kernel<T>, dim3(n), dim3(256), 0, (cudaStream_t)stream, x, w, (T*)y, rows, d, eps)));
    }
    return kp_launch_status();
}

// o: [n, ldo] float32, `groups` parts of `width` columns from column 0; g and out in the storage type `dtype`.
int kp_group_norm_gate_rows(const float* o, int ldo, const float* w, const void* g, int ldg, void* out, int ldout, int n, int groups,
                            int width, float eps, int gate_first, int gate_act, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (groups < 1 || width < 1 || gate_act < 0 || gate_act > 1) return KP_ERR_BAD_ARG;
    if (groups > 65535) return KP_ERR_UNSUPPORTED;
    {
        const int esz = dtype == KP_DTYPE_F32 ? 4 : 2;
        const bool aligned = width % 4 == 0 && ldo % 4 == 0 && ldg % 4 == 0 && ldout % 4 == 0 && (uintptr_t)o % 16 == 0 &&
                             (!w || (uintptr_t)w % 16 == 0) && (uintptr_t)g % (4 * esz) == 0 && (uintptr_t)out % (4 * esz) == 0;
        const long long items = (long long)n * groups;
        if (aligned && width <= 4096 && items < (1ll << 31)) {
            if (width <= 512) {
                KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(group_norm_gate_rows_vec_kernel<T, 32>, dim3((unsigned)((items + 7) / 8)), dim3(256), 0,
                                                           (cudaStream_t)stream, o, ldo, w, (const T*)g, ldg, (T*)out, ldout, (int)items,
                                                           groups, width, eps, gate_first, gate_act)));
            } else {
                KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(group_norm_gate_rows_vec_kernel<T, 256>, dim3((unsigned)items), dim3(256), 0,
                                                           (cudaStream_t)stream, o, ldo, w, (const T*)g, ldg, (T*)out, ldout, (int)items,
                                                           groups, width, eps, gate_first, gate_act)));
            }
            return kp_launch_status();
        }
    }
    const int threads = width >= 256 ? 256 : ((width + 31) / 32) * 32;      // by the part's width alone
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(group_norm_gate_rows_kernel<T>, dim3(n, groups), dim3(threads), 0, (cudaStream_t)stream, o,
                                               ldo, w, (const T*)g, ldg, (T*)out, ldout, width, eps, gate_first, gate_act)));
    return kp_launch_status();
}

int kp_head_gate(void* o, int ldo, const void* g, int ldg, int n, int H, int hd, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (H < 1 || hd < 1) return KP_ERR_BAD_ARG;
    const int esz = dtype == KP_DTYPE_F32 ? 4 : 2;
    if (hd % 4 == 0 && ldo % 4 == 0 && (uintptr_t)o % (4 * esz) == 0) {
        const int gv = grid_for((size_t)n * H * hd / 4, 256);
        KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(head_gate_vec_kernel<T>, dim3(gv), dim3(256), 0, (cudaStream_t)stream, (T*)o, ldo,
                                                   (const T*)g, ldg, n, H, hd)));
        return kp_launch_status();
    }
    const int gr = grid_for((size_t)n * H * hd, 256);
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(head_gate_kernel<T>, dim3(gr), dim3(256), 0, (cudaStream_t)stream, (T*)o, ldo, (const T*)g,
                                               ldg, n, H, hd)));
    return kp_launch_status();
}

int kp_softcap(float* x, long long n, float cap, void* stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.f)) return KP_ERR_BAD_ARG;
    kp_launch_pdl(softcap_kernel, dim3(grid_for((size_t)n, 256)), dim3(256), 0, (cudaStream_t)stream, x, (size_t)n, cap);
    return kp_launch_status();
}

int kp_glu_clamped(const void* gate_up, void* act, int n, int ff, float limit, float alpha, float shift, int dtype, void* stream) {
    if (n <= 0) return 0;
    const int g = grid_for((size_t)n * ff, 256);
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(glu_clamped_kernel<T>, dim3(g), dim3(256), 0, (cudaStream_t)stream, (const T*)gate_up, (T*)act,
                                               n, ff, limit, alpha, shift)));
    return kp_launch_status();
}

}  // extern "C"
