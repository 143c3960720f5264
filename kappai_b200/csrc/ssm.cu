// A selective state space mixer ("mamba2"): a short causal convolution with bias and silu over the channels
// [x | B | C] of one wide projection row, then, for every head h (reading group g(h) of B and C), the recurrence
//
//   dt_t = softplus(dt_raw_t + dt_bias_h)                       (no clamp; computed as max(z, 0) + log1p(exp(-|z|)))
//   S_t  = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T     (S: [state, vdim], float32, one a request and layer)
//   y_t  = S_t^T C_t + D_h x_t
//
// Everything of the recurrence is float32: step sizes, decays and their logarithms, the state, products and sums; the
// storage type holds the projection and the convolution's output only.  A request keeps, between steps, the state S
// and the last taps - 1 inputs of the convolution (both float32, in its slot; both count as zero at position 0).
//
// Kernels: the convolution (one thread a (row, channel), or 16 bytes of channels of four rows where the rows allow it;
// the same launch computes dt and the decay's logarithm of every (row, head)); the update of the kept inputs (a launch of its own behind it, because rows at a segment's head still
// read the old ones; in a step of single-row segments the convolution does it itself); the scan (a block walks the
// rows of one (segment, head, 16 value columns) with the state in registers, every sum in an order fixed by the sizes
// alone, so a row's bits do not depend on how the sequence was cut); and the chunked form for prompt portions in 16-bit
// mode (below).
#include "common.cuh"

#define SS_MAX_TAPS 16

__device__ __forceinline__ float ss_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float ss_softplus(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// p: rows [n, ld] in the storage type, the convolved channels at column conv_col (C of them), dt behind at dt_col (H).
// kept: [slots][slot_stride] float32, a slot's inputs as [taps - 1][C], oldest first.  out: [n, C] in the storage type.
// dt_out, da_out: [n, H] float32 (step size; logarithm of the decay).  fused_state: every segment has one row, and the
// thread that read a channel's kept inputs writes the new ones.
template <typename T>
__global__ void __launch_bounds__(128)
ssm_conv_kernel(const T* __restrict__ p, int ld, int conv_col, int dt_col, const float* __restrict__ taps,
                const float* __restrict__ bias, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                float* __restrict__ kept, size_t slot_stride, const int* __restrict__ row_seg, const int* __restrict__ cu_rows,
                const int* __restrict__ seg_pos, const int* __restrict__ seg_slot, T* __restrict__ out, float* __restrict__ dt_out,
                float* __restrict__ da_out, int C, int H, int K, int fused_state) {
    kp_pdl_begin();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (c >= C + H) return;
    if (c >= C) {
        const int h = c - C;
        const float dt = ss_softplus(to_f32(p[(size_t)r * ld + dt_col + h]) + dt_bias[h]);
        dt_out[(size_t)r * H + h] = dt;
        da_out[(size_t)r * H + h] = -expf(a_log[h]) * dt;
        return;
    }
    const int seg = row_seg[r], row0 = cu_rows[seg];
    const bool fresh = seg_pos[seg] == 0;
    float* kp = kept + (size_t)seg_slot[seg] * slot_stride;
    float acc = bias[c];
    float in[SS_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < SS_MAX_TAPS; j++) {
        if (j < K) {
            const int rr = r - (K - 1) + j;
            float v;
            if (rr >= row0) v = to_f32(p[(size_t)rr * ld + conv_col + c]);
            else v = fresh ? 0.f : kp[(size_t)(rr - row0 + K - 1) * C + c];
            in[j] = v;
            acc = fmaf(taps[(size_t)c * K + j], v, acc);
        }
    }
    out[(size_t)r * C + c] = from_f32<T>(ss_silu(acc));
    if (fused_state) {
#pragma unroll
        for (int j = 0; j < SS_MAX_TAPS - 1; j++)
            if (j < K - 1) kp[(size_t)j * C + c] = in[j + 1];
    }
}

// The same for prompt portions where rows and channels start on 16 bytes and K <= 4: a thread takes 16 bytes of
// channels (VW of them) of SV_ROWS consecutive rows and fetches every row of p once for all of them.  Every output is
// the same chain of multiply-adds as above (bias, then the taps from the oldest), so a row's bits do not depend on
// which form ran.  The last blocks along x compute dt and the decay's logarithm of the tile's rows.
#define SV_ROWS 4
template <typename T> struct SsVec;
template <> struct SsVec<bf16> {
    static constexpr int W = 8;
    __device__ static void load(const bf16* src, float* v) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(src));
        const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = __bfloat162float(e[i]);
    }
    __device__ static void store(bf16* dst, const float* v) {
        uint4 o;
        __nv_bfloat162 t;
        t = __floats2bfloat162_rn(v[0], v[1]); o.x = *reinterpret_cast<uint32_t*>(&t);
        t = __floats2bfloat162_rn(v[2], v[3]); o.y = *reinterpret_cast<uint32_t*>(&t);
        t = __floats2bfloat162_rn(v[4], v[5]); o.z = *reinterpret_cast<uint32_t*>(&t);
        t = __floats2bfloat162_rn(v[6], v[7]); o.w = *reinterpret_cast<uint32_t*>(&t);
        *reinterpret_cast<uint4*>(dst) = o;
    }
};
template <> struct SsVec<float> {
    static constexpr int W = 4;
    __device__ static void load(const float* src, float* v) {
        const float4 r = __ldg(reinterpret_cast<const float4*>(src));
        v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
    }
    __device__ static void store(float* dst, const float* v) { *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]); }
};

template <typename T, int K>
__global__ void __launch_bounds__(128)
ssm_conv_vec_kernel(const T* __restrict__ p, int ld, int conv_col, int dt_col, const float* __restrict__ taps,
                    const float* __restrict__ bias, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                    const float* __restrict__ kept, size_t slot_stride, const int* __restrict__ row_seg,
                    const int* __restrict__ cu_rows, const int* __restrict__ seg_pos, const int* __restrict__ seg_slot,
                    T* __restrict__ out, float* __restrict__ dt_out, float* __restrict__ da_out, int n, int C, int H, int conv_blocks) {
    kp_pdl_begin();
    constexpr int W = SsVec<T>::W;
    const int r0 = blockIdx.y * SV_ROWS;
    if ((int)blockIdx.x >= conv_blocks) {
        for (int x = (blockIdx.x - conv_blocks) * blockDim.x + threadIdx.x; x < SV_ROWS * H; x += (gridDim.x - conv_blocks) * blockDim.x) {
            const int r = r0 + x / H, h = x % H;
            if (r < n) {
                const float dt = ss_softplus(to_f32(p[(size_t)r * ld + dt_col + h]) + dt_bias[h]);
                dt_out[(size_t)r * H + h] = dt;
                da_out[(size_t)r * H + h] = -expf(a_log[h]) * dt;
            }
        }
        return;
    }
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * W;
    if (c >= C) return;
    // rows r0 - (K - 1) .. r0 + SV_ROWS - 1 of this step (zero where there is none; whether a row counts is decided below)
    float win[SV_ROWS + K - 1][W];
#pragma unroll
    for (int i = 0; i < SV_ROWS + K - 1; i++) {
        const int rr = r0 - (K - 1) + i;
        if (rr >= 0 && rr < n) SsVec<T>::load(p + (size_t)rr * ld + conv_col + c, win[i]);
        else {
#pragma unroll
            for (int e = 0; e < W; e++) win[i][e] = 0.f;
        }
    }
    // the thread's W K taps lie side by side and start on 32 bytes (c is a multiple of W): 16 bytes a load
    float tp[W][K], bs[W];
    {
        float flat[W * K];
        const float4* t4 = reinterpret_cast<const float4*>(taps + (size_t)c * K);
#pragma unroll
        for (int i = 0; i < W * K / 4; i++) {
            const float4 t = __ldg(t4 + i);
            flat[4 * i] = t.x; flat[4 * i + 1] = t.y; flat[4 * i + 2] = t.z; flat[4 * i + 3] = t.w;
        }
        const float4* b4 = reinterpret_cast<const float4*>(bias + c);
#pragma unroll
        for (int i = 0; i < W / 4; i++) {
            const float4 t = __ldg(b4 + i);
            bs[4 * i] = t.x; bs[4 * i + 1] = t.y; bs[4 * i + 2] = t.z; bs[4 * i + 3] = t.w;
        }
#pragma unroll
        for (int e = 0; e < W; e++)
#pragma unroll
            for (int j = 0; j < K; j++) tp[e][j] = flat[e * K + j];
    }
#pragma unroll
    for (int i = 0; i < SV_ROWS; i++) {
        const int r = r0 + i;
        if (r >= n) break;
        const int seg = row_seg[r], row0 = cu_rows[seg];
        const bool fresh = seg_pos[seg] == 0;
        const float* kp = kept + (size_t)seg_slot[seg] * slot_stride;
        float acc[W];
#pragma unroll
        for (int e = 0; e < W; e++) acc[e] = bs[e];
#pragma unroll
        for (int j = 0; j < K; j++) {
            const int rr = r - (K - 1) + j;
            if (rr >= row0) {
#pragma unroll
                for (int e = 0; e < W; e++) acc[e] = fmaf(tp[e][j], win[i + j][e], acc[e]);
            } else if (!fresh) {
                const float* kr = kp + (size_t)(rr - row0 + K - 1) * C + c;
#pragma unroll
                for (int e = 0; e < W; e++) acc[e] = fmaf(tp[e][j], kr[e], acc[e]);
            } else {
#pragma unroll
                for (int e = 0; e < W; e++) acc[e] = fmaf(tp[e][j], 0.f, acc[e]);
            }
        }
#pragma unroll
        for (int e = 0; e < W; e++) acc[e] = ss_silu(acc[e]);
        SsVec<T>::store(out + (size_t)r * C + c, acc);
    }
}

// The inputs a request keeps behind a segment of len rows: its last taps - 1, from the rows of this step and, where the
// segment is shorter than that, from what was kept before (zero for a fresh sequence).
template <typename T>
__global__ void __launch_bounds__(128)
ssm_conv_keep_kernel(const T* __restrict__ p, int ld, int conv_col, float* __restrict__ kept, size_t slot_stride,
                     const int* __restrict__ cu_rows, const int* __restrict__ seg_pos, const int* __restrict__ seg_slot, int C, int K) {
    kp_pdl_begin();
    const int seg = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int row0 = cu_rows[seg], row1 = cu_rows[seg + 1], len = row1 - row0;
    const bool fresh = seg_pos[seg] == 0;
    float* kp = kept + (size_t)seg_slot[seg] * slot_stride;
    for (int j = 0; j < K - 1; j++) {                       // ascending: index len + j is read before it is written
        const int rr = row1 - (K - 1) + j;
        float v;
        if (rr >= row0) v = to_f32(p[(size_t)rr * ld + conv_col + c]);
        else v = fresh ? 0.f : kp[(size_t)(len + j) * C + c];
        kp[(size_t)j * C + c] = v;
    }
}

// ------------------------------------------------------------------------------------------------ the scan
#define SS_CH_MAX 16             // rows staged at a time (half as many for the largest states: shared memory)
#define SS_COLS 16               // value columns of a block
#define SS_PARTS 16              // parts the state's rows are cut in
#define SS_THREADS (SS_COLS * SS_PARTS)

// R: state rows a thread keeps (N <= SS_PARTS * R).  Thread (part q, column c) owns rows q R .. q R + R - 1 of column c.
// xbc: [n, ldx] in the storage type: x at column 0 (H heads of P), B at b_col, C at c_col (G groups of N each).
template <typename T, int R>
__global__ void __launch_bounds__(SS_THREADS)
ssm_scan_kernel(const T* __restrict__ xbc, int ldx, int b_col, int c_col, const float* __restrict__ dt, const float* __restrict__ da,
                const float* __restrict__ Dh, float* __restrict__ state, size_t slot_stride, const int* __restrict__ cu_rows,
                const int* __restrict__ seg_pos, const int* __restrict__ seg_slot, float* __restrict__ y, int ldy, int H, int G,
                int N, int P, int write_state) {
    kp_pdl_begin();
    constexpr int NP = SS_PARTS * R;
    constexpr int CH = R >= 16 ? SS_CH_MAX / 2 : SS_CH_MAX;
    __shared__ __align__(16) float sb[CH][NP];               // dt_t B_t
    __shared__ __align__(16) float sc[CH][NP];               // C_t
    __shared__ float sx[CH][SS_COLS];
    __shared__ float sa[CH];
    __shared__ float part[CH][SS_PARTS][SS_COLS];
    const int seg = blockIdx.x, head = blockIdx.y, tile = blockIdx.z;
    const int grp = head / (H / G);
    const int c = threadIdx.x & (SS_COLS - 1), q = threadIdx.x / SS_COLS;
    const int j = tile * SS_COLS + c;
    const bool jok = j < P;
    const float dskip = Dh[head];
    float* st = state + (size_t)seg_slot[seg] * slot_stride + ((size_t)head * N) * P;
    float s[R];
    const bool fresh = seg_pos[seg] == 0;
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int i = q * R + r;
        s[r] = (!fresh && jok && i < N) ? st[(size_t)i * P + j] : 0.f;
    }
    const int row0 = cu_rows[seg], row1 = cu_rows[seg + 1];
    for (int t0 = row0; t0 < row1; t0 += CH) {
        const int nt = min(CH, row1 - t0);
        __syncthreads();
        for (int x = threadIdx.x; x < nt * NP; x += SS_THREADS) {
            const int t = x / NP, i = x - t * NP;
            float bv = 0.f, cv = 0.f;
            if (i < N) {
                const T* row = xbc + (size_t)(t0 + t) * ldx + grp * N + i;
                bv = dt[(size_t)(t0 + t) * H + head] * to_f32(row[b_col]);
                cv = to_f32(row[c_col]);
            }
            sb[t][i] = bv;
            sc[t][i] = cv;
        }
        for (int x = threadIdx.x; x < nt * SS_COLS; x += SS_THREADS) {
            const int t = x / SS_COLS, l = x % SS_COLS, jj = tile * SS_COLS + l;
            sx[t][l] = jj < P ? to_f32(xbc[(size_t)(t0 + t) * ldx + head * P + jj]) : 0.f;
        }
        if (threadIdx.x < nt) sa[threadIdx.x] = expf(da[(size_t)(t0 + threadIdx.x) * H + head]);
        __syncthreads();
        for (int t = 0; t < nt; t++) {
            const float xj = sx[t][c], a = sa[t];
            const float* bt = &sb[t][q * R];
            const float* ct = &sc[t][q * R];
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < R; r++) {
                s[r] = fmaf(a, s[r], bt[r] * xj);
                acc = fmaf(s[r], ct[r], acc);
            }
            part[t][q][c] = acc;
        }
        __syncthreads();
        for (int x = threadIdx.x; x < nt * SS_COLS; x += SS_THREADS) {
            const int t = x / SS_COLS, l = x % SS_COLS, jj = tile * SS_COLS + l;
            float sum = part[t][0][l];
#pragma unroll
            for (int k = 1; k < SS_PARTS; k++) sum += part[t][k][l];
            if (jj < P) y[(size_t)(t0 + t) * ldy + head * P + jj] = fmaf(dskip, sx[t][l], sum);
        }
    }
    if (write_state && jok) {
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int i = q * R + r;
            if (i < N) st[(size_t)i * P + j] = s[r];
        }
    }
}

// ------------------------------------------------------------------------------------------------ chunked
// For prompt portions in 16-bit mode: a segment in chunks of SC_C rows.  With L_i the sum of the decays' logarithms
// from the chunk's first row up to row i, the rows of a chunk are independent given the state S at its head:
//   y_i = sum_{j <= i} exp(L_i - L_j) (C_i . B_j) dt_j x_j + exp(L_i) C_i^T S + D x_i ,
//   S'  = exp(L_last) S + sum_j exp(L_last - L_j) dt_j B_j x_j^T ,
// small float32 matrix products from shared memory.  The chunks of all segments run side by side: (0) the products
// C_i . B_j of every (chunk, group), which all heads of the group share, (1) every chunk's own sum U_c and its whole
// decay, (2) a serial pass a (segment, head) that turns the sums into the states at the chunks' heads in place and
// leaves the last state in the slot, (3) every chunk's outputs.  Every exponent is <= 0.
#define SC_C 64
#define SC_LD (SC_C + 4)
#define SC_COLS 32
#define SC_THREADS 256
#define SC_MAX_N 128

// L_i of the chunk's rows into shared memory (a serial sum by one thread: 64 additions, the same order every time).
__device__ __forceinline__ void sc_prefix(float* L, const float* __restrict__ da, int H, int head, int t0, int n, int tid) {
    if (tid == 0) {
        float acc = 0.f;
        for (int t = 0; t < n; t++) {
            acc += da[(size_t)(t0 + t) * H + head];
            L[t] = acc;
        }
    }
}

// A [rows t0 .. t0 + n) x [N] stretch of columns transposed into dst [N][SC_LD] (zeros behind the n rows).
// vec: the stretch starts on 16 bytes in every row and N is a multiple of 8 (bfloat16 rows): 16 bytes a load.
template <typename T>
__device__ __forceinline__ void sc_stage_transposed(float* dst, const T* __restrict__ xbc, int ldx, int col, int N, int t0, int n, int tid,
                                                    bool vec) {
    if (sizeof(T) == 2 && vec) {
        const int ng = N / 8;
        for (int x = tid; x < ng * SC_C; x += SC_THREADS) {
            const int t = x % SC_C, g = x / SC_C;
            uint4 raw = make_uint4(0u, 0u, 0u, 0u);
            if (t < n) raw = __ldg(reinterpret_cast<const uint4*>(xbc + (size_t)(t0 + t) * ldx + col + g * 8));
            const bf16* e8 = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
            for (int e = 0; e < 8; e++) dst[(g * 8 + e) * SC_LD + t] = __bfloat162float(e8[e]);
        }
        return;
    }
    for (int x = tid; x < N * SC_C; x += SC_THREADS) {
        const int t = x % SC_C, d = x / SC_C;
        dst[d * SC_LD + t] = t < n ? to_f32(xbc[(size_t)(t0 + t) * ldx + col + d]) : 0.f;
    }
}

template <typename T>
__device__ __forceinline__ void sc_stage_values(float* Vs, const T* __restrict__ xbc, int ldx, int head, int P, int tile, int t0, int n, int tid) {
    for (int x = tid; x < SC_C * SC_COLS; x += SC_THREADS) {
        const int t = x / SC_COLS, c = x % SC_COLS, j = tile * SC_COLS + c;
        Vs[x] = (t < n && j < P) ? to_f32(xbc[(size_t)(t0 + t) * ldx + head * P + j]) : 0.f;
    }
}

// (1) U[chunk][head] = sum_j exp(L_last - L_j) dt_j B_j x_j^T ;  cdec[chunk][head] = exp(L_last)
template <typename T>
__global__ void __launch_bounds__(SC_THREADS)
ssm_chunk_sums_kernel(const T* __restrict__ xbc, int ldx, int b_col, const float* __restrict__ dt, const float* __restrict__ da,
                      const int* __restrict__ cu_rows, const int* __restrict__ chunk_seg, const int* __restrict__ chunk_row0,
                      float* __restrict__ U, float* __restrict__ cdec, int H, int G, int N, int P, int vec) {
    kp_pdl_begin();
    extern __shared__ __align__(16) float sc_sm[];
    float* Bt = sc_sm;                                           // [N][SC_LD]
    float* Vs = Bt + (size_t)N * SC_LD;                          // [SC_C][SC_COLS]
    float* L = Vs + SC_C * SC_COLS;                              // [SC_C]
    float* kw = L + SC_C;                                        // [SC_C]
    const int chunk = blockIdx.x, head = blockIdx.y, tile = blockIdx.z, tid = threadIdx.x;
    const int grp = head / (H / G);
    const int t0 = chunk_row0[chunk], n = min(SC_C, cu_rows[chunk_seg[chunk] + 1] - t0);
    sc_prefix(L, da, H, head, t0, n, tid);
    sc_stage_transposed<T>(Bt, xbc, ldx, b_col + grp * N, N, t0, n, tid, vec != 0);
    sc_stage_values<T>(Vs, xbc, ldx, head, P, tile, t0, n, tid);
    __syncthreads();
    for (int x = tid; x < SC_C; x += SC_THREADS) kw[x] = x < n ? expf(L[n - 1] - L[x]) * dt[(size_t)(t0 + x) * H + head] : 0.f;
    if (tid == 0 && tile == 0) cdec[(size_t)chunk * H + head] = expf(L[n - 1]);
    __syncthreads();
    const int r0 = (tid / 8) * 2, c0 = (tid % 8) * 4;
    float* Uc = U + ((size_t)chunk * H + head) * N * P;
    for (int d0 = r0; d0 < N; d0 += 2 * (SC_THREADS / 8)) {
        float acc[2][4];
#pragma unroll
        for (int a = 0; a < 2; a++)
#pragma unroll
            for (int b = 0; b < 4; b++) acc[a][b] = 0.f;
        const bool two = d0 + 1 < N;
#pragma unroll 4
        for (int j = 0; j < n; j++) {
            const float w = kw[j];
            const float k0 = Bt[d0 * SC_LD + j] * w, k1 = two ? Bt[(d0 + 1) * SC_LD + j] * w : 0.f;
            const float4 v4 = *reinterpret_cast<const float4*>(Vs + j * SC_COLS + c0);
            acc[0][0] = fmaf(k0, v4.x, acc[0][0]); acc[0][1] = fmaf(k0, v4.y, acc[0][1]);
            acc[0][2] = fmaf(k0, v4.z, acc[0][2]); acc[0][3] = fmaf(k0, v4.w, acc[0][3]);
            acc[1][0] = fmaf(k1, v4.x, acc[1][0]); acc[1][1] = fmaf(k1, v4.y, acc[1][1]);
            acc[1][2] = fmaf(k1, v4.z, acc[1][2]); acc[1][3] = fmaf(k1, v4.w, acc[1][3]);
        }
#pragma unroll
        for (int a = 0; a < 2; a++) {
            if (d0 + a >= N) continue;
#pragma unroll
            for (int b = 0; b < 4; b++) {
                const int j = tile * SC_COLS + c0 + b;
                if (j < P) Uc[(size_t)(d0 + a) * P + j] = acc[a][b];
            }
        }
    }
}

// (2) in place: U[chunk] <- the state at the chunk's head; the segment's slot <- the state behind its last chunk
__global__ void __launch_bounds__(256)
ssm_chunk_states_kernel(float* __restrict__ U, const float* __restrict__ cdec, float* __restrict__ state, size_t slot_stride,
                        const int* __restrict__ seg_pos, const int* __restrict__ seg_slot, const int* __restrict__ seg_chunk0,
                        int H, int N, int P, int write_state) {
    kp_pdl_begin();
    const int seg = blockIdx.x, head = blockIdx.y;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    if (e >= N * P) return;
    float* st = state + (size_t)seg_slot[seg] * slot_stride + (size_t)head * N * P + e;
    float S = seg_pos[seg] == 0 ? 0.f : *st;
    const size_t stride = (size_t)H * N * P;
    const int c_end = seg_chunk0[seg + 1];
    for (int c0 = seg_chunk0[seg]; c0 < c_end; c0 += 8) {
        float* p = U + ((size_t)c0 * H + head) * N * P + e;
        float u[8], w[8];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            if (c0 + k < c_end) {
                u[k] = p[k * stride];
                w[k] = cdec[(size_t)(c0 + k) * H + head];
            }
        }
#pragma unroll
        for (int k = 0; k < 8; k++) {
            if (c0 + k < c_end) {
                p[k * stride] = S;
                S = fmaf(w[k], S, u[k]);
            }
        }
    }
    if (write_state) *st = S;
}

// (0) M[chunk][group][i][j] = C_i . B_j for the 4 x 4 pieces of the chunk that hold a j <= i: the same for all heads of a
// group and all tiles of their values, so it is computed once.
template <typename T>
__global__ void __launch_bounds__(SC_THREADS)
ssm_chunk_cb_kernel(const T* __restrict__ xbc, int ldx, int b_col, int c_col, const int* __restrict__ cu_rows,
                    const int* __restrict__ chunk_seg, const int* __restrict__ chunk_row0, float* __restrict__ M, int G, int N, int vec) {
    kp_pdl_begin();
    extern __shared__ __align__(16) float sc_sm[];
    float* Ct = sc_sm;                                           // [N][SC_LD]
    float* Bt = Ct + (size_t)N * SC_LD;                          // [N][SC_LD]
    const int chunk = blockIdx.x, grp = blockIdx.y, tid = threadIdx.x;
    const int t0 = chunk_row0[chunk], n = min(SC_C, cu_rows[chunk_seg[chunk] + 1] - t0);
    sc_stage_transposed<T>(Ct, xbc, ldx, c_col + grp * N, N, t0, n, tid, vec != 0);
    sc_stage_transposed<T>(Bt, xbc, ldx, b_col + grp * N, N, t0, n, tid, vec != 0);
    __syncthreads();
    const int i0 = (tid / 16) * 4, j0 = (tid % 16) * 4;
    if (!(j0 <= i0 + 3 && i0 < n)) return;
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
        for (int b = 0; b < 4; b++) acc[a][b] = 0.f;
#pragma unroll 4
    for (int d = 0; d < N; d++) {
        const float4 q4 = *reinterpret_cast<const float4*>(Ct + d * SC_LD + i0);
        const float4 k4 = *reinterpret_cast<const float4*>(Bt + d * SC_LD + j0);
        const float qa[4] = {q4.x, q4.y, q4.z, q4.w}, kb[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
        for (int a = 0; a < 4; a++)
#pragma unroll
            for (int b = 0; b < 4; b++) acc[a][b] = fmaf(qa[a], kb[b], acc[a][b]);
    }
    float* Mc = M + ((size_t)chunk * G + grp) * SC_C * SC_C;
#pragma unroll
    for (int a = 0; a < 4; a++)
        *reinterpret_cast<float4*>(Mc + (i0 + a) * SC_C + j0) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
}

// (3) y_i = sum_{j <= i} exp(L_i - L_j) (C_i . B_j) dt_j x_j + exp(L_i) C_i^T S + D x_i, S the state at the chunk's head;
// the products C_i . B_j come from pass (0)
template <typename T>
__global__ void __launch_bounds__(SC_THREADS)
ssm_chunk_out_kernel(const T* __restrict__ xbc, int ldx, int c_col, const float* __restrict__ dt, const float* __restrict__ da,
                     const float* __restrict__ Dh, const int* __restrict__ cu_rows, const int* __restrict__ chunk_seg,
                     const int* __restrict__ chunk_row0, const float* __restrict__ U, const float* __restrict__ M, float* __restrict__ y,
                     int ldy, int H, int G, int N, int P, int vec) {
    kp_pdl_begin();
    extern __shared__ __align__(16) float sc_sm[];
    float* Ct = sc_sm;                                           // [N][SC_LD]
    float* Vs = Ct + (size_t)N * SC_LD;                          // [SC_C][SC_COLS]
    float* Ps = Vs + SC_C * SC_COLS;                             // [SC_C][SC_LD]
    float* Ss = Ps + SC_C * SC_LD;                               // [N][SC_COLS]
    float* L = Ss + (size_t)N * SC_COLS;                         // [SC_C]
    float* dts = L + SC_C;                                       // [SC_C]
    const int chunk = blockIdx.x, head = blockIdx.y, tile = blockIdx.z, tid = threadIdx.x;
    const int grp = head / (H / G);
    const int t0 = chunk_row0[chunk], n = min(SC_C, cu_rows[chunk_seg[chunk] + 1] - t0);
    sc_prefix(L, da, H, head, t0, n, tid);
    sc_stage_transposed<T>(Ct, xbc, ldx, c_col + grp * N, N, t0, n, tid, vec != 0);
    sc_stage_values<T>(Vs, xbc, ldx, head, P, tile, t0, n, tid);
    const float* Sc = U + ((size_t)chunk * H + head) * N * P;
    for (int x = tid; x < N * SC_COLS; x += SC_THREADS) {
        const int d = x / SC_COLS, c = x % SC_COLS, j = tile * SC_COLS + c;
        Ss[x] = j < P ? Sc[(size_t)d * P + j] : 0.f;
    }
    for (int x = tid; x < SC_C; x += SC_THREADS) dts[x] = x < n ? dt[(size_t)(t0 + x) * H + head] : 0.f;
    __syncthreads();
    if (tid >= n && tid < SC_C) L[tid] = 0.f;
    __syncthreads();
    const int i0 = (tid / 16) * 4, j0 = (tid % 16) * 4;
    const int r0 = (tid / 8) * 2, c0 = (tid % 8) * 4;
    {
        const bool piece = j0 <= i0 + 3 && i0 < n;                // (the pieces that pass (0) wrote)
        const float* Mc = M + ((size_t)chunk * G + grp) * SC_C * SC_C;
#pragma unroll
        for (int a = 0; a < 4; a++) {
            float4 m4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (piece) m4 = *reinterpret_cast<const float4*>(Mc + (i0 + a) * SC_C + j0);
            const float ma[4] = {m4.x, m4.y, m4.z, m4.w};
            float4 out;
            float* po = reinterpret_cast<float*>(&out);
#pragma unroll
            for (int b = 0; b < 4; b++) {
                const int i = i0 + a, j = j0 + b;
                po[b] = (j <= i && i < n) ? ma[b] * (expf(L[i] - L[j]) * dts[j]) : 0.f;
            }
            *reinterpret_cast<float4*>(Ps + (i0 + a) * SC_LD + j0) = out;
        }
    }
    __syncthreads();
    if (r0 >= n) return;
    float ap[2][4], as[2][4];
#pragma unroll
    for (int a = 0; a < 2; a++)
#pragma unroll
        for (int b = 0; b < 4; b++) { ap[a][b] = 0.f; as[a][b] = 0.f; }
    const int jn = min(n, r0 + 2);
#pragma unroll 4
    for (int j = 0; j < jn; j++) {
        const float p0 = Ps[r0 * SC_LD + j], p1 = Ps[(r0 + 1) * SC_LD + j];
        const float4 v4 = *reinterpret_cast<const float4*>(Vs + j * SC_COLS + c0);
        ap[0][0] = fmaf(p0, v4.x, ap[0][0]); ap[0][1] = fmaf(p0, v4.y, ap[0][1]);
        ap[0][2] = fmaf(p0, v4.z, ap[0][2]); ap[0][3] = fmaf(p0, v4.w, ap[0][3]);
        ap[1][0] = fmaf(p1, v4.x, ap[1][0]); ap[1][1] = fmaf(p1, v4.y, ap[1][1]);
        ap[1][2] = fmaf(p1, v4.z, ap[1][2]); ap[1][3] = fmaf(p1, v4.w, ap[1][3]);
    }
#pragma unroll 4
    for (int d = 0; d < N; d++) {
        const float2 q2 = *reinterpret_cast<const float2*>(Ct + d * SC_LD + r0);
        const float4 s4 = *reinterpret_cast<const float4*>(Ss + d * SC_COLS + c0);
        as[0][0] = fmaf(q2.x, s4.x, as[0][0]); as[0][1] = fmaf(q2.x, s4.y, as[0][1]);
        as[0][2] = fmaf(q2.x, s4.z, as[0][2]); as[0][3] = fmaf(q2.x, s4.w, as[0][3]);
        as[1][0] = fmaf(q2.y, s4.x, as[1][0]); as[1][1] = fmaf(q2.y, s4.y, as[1][1]);
        as[1][2] = fmaf(q2.y, s4.z, as[1][2]); as[1][3] = fmaf(q2.y, s4.w, as[1][3]);
    }
    const float dskip = Dh[head];
#pragma unroll
    for (int a = 0; a < 2; a++) {
        const int i = r0 + a;
        if (i >= n) continue;
        const float w = expf(L[i]);
        float* dst = y + (size_t)(t0 + i) * ldy + head * P + tile * SC_COLS + c0;
#pragma unroll
        for (int b = 0; b < 4; b++)
            if (tile * SC_COLS + c0 + b < P) dst[b] = fmaf(dskip, Vs[i * SC_COLS + c0 + b], fmaf(w, as[a][b], ap[a][b]));
    }
}

extern "C" {

// The convolution with bias and silu over the C channels at conv_col of p, dt and the decay's logarithm of the H heads
// at dt_col.  taps [C][K], bias [C], dt_bias, a_log [H].  kept: a slot's last K - 1 inputs at `kept + slot *
// slot_stride`.  single_rows != 0: every segment has one row and the kept inputs are renewed here; else they are
// renewed by a second launch behind the first unless keep == 0.
int kp_ssm_conv(const void* p, int ld, int conv_col, int dt_col, const float* taps, const float* bias, const float* dt_bias,
                const float* a_log, float* kept, long long slot_stride, const int* row_seg, const int* cu_rows, const int* seg_pos,
                const int* seg_slot, void* out, float* dt_out, float* da_out, int n, int n_seg, int C, int H, int K, int single_rows,
                int keep, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (C < 1 || H < 1 || K < 1 || K > SS_MAX_TAPS || n > 65535 || n_seg > 65535) return KP_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int fused = single_rows && keep;
    const int vw = dtype == KP_DTYPE_F32 ? 4 : 8;
    const bool vec = !single_rows && K <= 4 && n >= 2 * SV_ROWS && C % vw == 0 && ld % vw == 0 && conv_col % vw == 0 &&
                     (uintptr_t)p % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)taps % 16 == 0 && (uintptr_t)bias % 16 == 0;
    if (vec) {
        const int conv_blocks = (C / vw + 127) / 128, dt_blocks = (SV_ROWS * H + 127) / 128 > 4 ? 4 : (SV_ROWS * H + 127) / 128;
        const dim3 grid(conv_blocks + dt_blocks, (n + SV_ROWS - 1) / SV_ROWS);
#define SV_LAUNCH(KK)                                                                                                        \
        KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(ssm_conv_vec_kernel<T, KK>, grid, dim3(128), 0, s, (const T*)p, ld, conv_col, dt_col, taps,  \
                                                   bias, dt_bias, a_log, (const float*)kept, (size_t)slot_stride, row_seg, cu_rows, seg_pos, \
                                                   seg_slot, (T*)out, dt_out, da_out, n, C, H, conv_blocks)))
        if (K == 1) SV_LAUNCH(1); else if (K == 2) SV_LAUNCH(2); else if (K == 3) SV_LAUNCH(3); else SV_LAUNCH(4);
#undef SV_LAUNCH
    } else {
        KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(ssm_conv_kernel<T>, dim3((C + H + 127) / 128, n), dim3(128), 0, s, (const T*)p, ld, conv_col,
                                                   dt_col, taps, bias, dt_bias, a_log, kept, (size_t)slot_stride, row_seg, cu_rows, seg_pos,
                                                   seg_slot, (T*)out, dt_out, da_out, C, H, K, fused)));
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (keep && !fused && K > 1) {
        KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(ssm_conv_keep_kernel<T>, dim3((C + 127) / 128, n_seg), dim3(128), 0, s, (const T*)p, ld,
                                                   conv_col, kept, (size_t)slot_stride, cu_rows, seg_pos, seg_slot, C, K)));
    }
    return kp_launch_status();
}

// xbc: [n, ldx] in the storage type (x: H heads of P at column 0; B at b_col, C at c_col: G groups of N).  dt, da: [n, H]
// float32.  state: a slot's [H][N][P] float32 at `state + slot * slot_stride`.  y: [n, ldy] float32, heads side by side.
int kp_ssm_scan(const void* xbc, int ldx, int b_col, int c_col, const float* dt, const float* da, const float* Dh, float* state,
                long long slot_stride, const int* cu_rows, const int* seg_pos, const int* seg_slot, float* y, int ldy, int n_seg,
                int H, int G, int N, int P, int write_state, int dtype, void* stream) {
    if (n_seg <= 0) return 0;
    if (H < 1 || G < 1 || H % G || N < 1 || P < 1) return KP_ERR_BAD_ARG;
    if (N > 16 * SS_PARTS || H > 65535 || (P + SS_COLS - 1) / SS_COLS > 65535) return KP_ERR_UNSUPPORTED;
    const dim3 grid(n_seg, H, (P + SS_COLS - 1) / SS_COLS), block(SS_THREADS);
    cudaStream_t s = (cudaStream_t)stream;
#define SS_LAUNCH(T, R)                                                                                                      \
    kp_launch_pdl(ssm_scan_kernel<T, R>, grid, block, 0, s, (const T*)xbc, ldx, b_col, c_col, dt, da, Dh, state, (size_t)slot_stride, \
                  cu_rows, seg_pos, seg_slot, y, ldy, H, G, N, P, write_state)
    // (the rows a thread keeps depend on the state's size only, so a row's sums have the same order in every launch)
    KP_DISPATCH_DTYPE(dtype, T, {
        if (N <= 2 * SS_PARTS) SS_LAUNCH(T, 2);
        else if (N <= 4 * SS_PARTS) SS_LAUNCH(T, 4);
        else if (N <= 8 * SS_PARTS) SS_LAUNCH(T, 8);
        else SS_LAUNCH(T, 16);
    });
#undef SS_LAUNCH
    return kp_launch_status();
}

int kp_ssm_chunk_rows() { return SC_C; }
// floats of scratch that kp_ssm_chunks wants: every chunk's sum a head, its decay, and the products C B^T a (chunk, group)
long long kp_ssm_chunks_scratch(int n_chunks, int H, int G, int N, int P) {
    return (((long long)n_chunks * H * N * P + (long long)n_chunks * H + 3) / 4) * 4 + (long long)n_chunks * G * SC_C * SC_C;
}

// The chunked form: the arguments of kp_ssm_scan and the list of chunks (chunk_seg, chunk_row0 [n_chunks]: every chunk's
// segment, numbered among the n_seg segments given here, and first row; seg_chunk0 [n_seg + 1]: the first chunk of every
// segment).  scratch: kp_ssm_chunks_scratch floats, 16-byte aligned.  KP_ERR_UNSUPPORTED for states it does not take (N > 128).
int kp_ssm_chunks(const void* xbc, int ldx, int b_col, int c_col, const float* dt, const float* da, const float* Dh, float* state,
                  long long slot_stride, const int* cu_rows, const int* seg_pos, const int* seg_slot, const int* chunk_seg,
                  const int* chunk_row0, const int* seg_chunk0, int n_chunks, float* scratch, float* y, int ldy, int n_seg, int H,
                  int G, int N, int P, int write_state, int dtype, void* stream) {
    if (n_seg <= 0 || n_chunks <= 0) return 0;
    if (H < 1 || G < 1 || H % G || N < 1 || P < 1) return KP_ERR_BAD_ARG;
    const int tiles = (P + SC_COLS - 1) / SC_COLS;
    if (N > SC_MAX_N || H > 65535 || tiles > 65535 || (N * P + 255) / 256 > 65535) return KP_ERR_UNSUPPORTED;
    const size_t sm0 = (size_t)2 * N * SC_LD * sizeof(float);
    const size_t sm1 = ((size_t)N * SC_LD + SC_C * SC_COLS + 2 * SC_C) * sizeof(float);
    const size_t sm3 = ((size_t)N * SC_LD + SC_C * SC_COLS + SC_C * SC_LD + (size_t)N * SC_COLS + 2 * SC_C) * sizeof(float);
    float* U = scratch;
    float* cdec = scratch + (size_t)n_chunks * H * N * P;
    float* M = scratch + (((size_t)n_chunks * H * N * P + (size_t)n_chunks * H + 3) / 4) * 4;      // (on 16 bytes behind both)
    const int esz = dtype == KP_DTYPE_F32 ? 4 : 2;
    const int vec = (esz == 2 && N % 8 == 0 && ldx % 8 == 0 && b_col % 8 == 0 && c_col % 8 == 0 && (uintptr_t)xbc % 16 == 0) ? 1 : 0;
    if ((uintptr_t)scratch % 16) return KP_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    KP_DISPATCH_DTYPE(dtype, T, {
        if ((e = cudaFuncSetAttribute(ssm_chunk_cb_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm0)) != cudaSuccess) return (int)e;
        if ((e = cudaFuncSetAttribute(ssm_chunk_sums_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm1)) != cudaSuccess) return (int)e;
        if ((e = cudaFuncSetAttribute(ssm_chunk_out_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm3)) != cudaSuccess) return (int)e;
        kp_launch_pdl(ssm_chunk_cb_kernel<T>, dim3(n_chunks, G), dim3(SC_THREADS), sm0, s, (const T*)xbc, ldx, b_col, c_col, cu_rows, chunk_seg,
                      chunk_row0, M, G, N, vec);
        if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
        kp_launch_pdl(ssm_chunk_sums_kernel<T>, dim3(n_chunks, H, tiles), dim3(SC_THREADS), sm1, s, (const T*)xbc, ldx, b_col, dt, da, cu_rows,
                      chunk_seg, chunk_row0, U, cdec, H, G, N, P, vec);
        if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
        kp_launch_pdl(ssm_chunk_states_kernel, dim3(n_seg, H, (N * P + 255) / 256), dim3(256), 0, s, U, (const float*)cdec, state,
                      (size_t)slot_stride, seg_pos, seg_slot, seg_chunk0, H, N, P, write_state);
        if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
        kp_launch_pdl(ssm_chunk_out_kernel<T>, dim3(n_chunks, H, tiles), dim3(SC_THREADS), sm3, s, (const T*)xbc, ldx, c_col, dt, da, Dh,
                      cu_rows, chunk_seg, chunk_row0, (const float*)U, (const float*)M, y, ldy, H, G, N, P, vec);
    });
    return kp_launch_status();
}

}  // extern "C"
