// Linear attention with a per-head decay ("lightning attention"), a recurrence over the tokens of a sequence:
//
//   S_t = a_h S_(t-1) + k_t v_t^T          (S: [dim, vdim] for every head, float32, one a request and layer)
//   o_t = S_t^T q_t
//
// with q, k, v = act(projection) (act = silu or none), read from columns of one wide row in the storage type.
// Optionally q and k are rotated by position as they are staged (the first `rot` dimensions of a head, dimension i
// paired with i + rot/2, cos and sin from tables [position][rot/2] made in double), and k is multiplied by a constant
// behind the rotation; both in float32, so that what enters the recurrence was never rounded to the storage type.
// Everything of the recurrence is float32: the state, the decay (carried as a float32 pair hi + lo so that a
// thousand steps of it do not drift from the constant the model gives), the products and the sums.  The state of a
// request lives in its slot between steps and counts as zero at position 0.
//
// Two forms.  The scan: a block walks the rows of one (segment, head, 16 value columns) in order, the state in
// registers (thread = (value column, a sixteenth of the key rows)); rows are staged 16 (or 8) at a time, q and k with
// their activation applied once, and a thread reads its stretch of them as float4.  One row a segment is the decode
// step.  Every sum has a fixed order that depends on the head's size alone, so a row's bits do not depend on how the
// sequence was cut or on what else is in the batch.
//
// The chunked form, for prompt portions in 16-bit mode: a segment in chunks of LC_C rows; within a chunk the rows are
// independent given the state S at its head,
//   o_i = sum_{j <= i} a^(i-j) (q_i . k_j) v_j + a^(i+1) q_i^T S ,     S' = a^n S + sum_j a^(n-1-j) k_j v_j^T ,
// three small float32 matrix products from shared memory (q and k staged transposed, so that every product reads
// its operands along rows) instead of LC_C dependent steps.  The chunks of all segments run side by side with a
// short serial pass between them (see "chunks in parallel" below).  The powers of the decay come from a table made
// in double on the host.  Sums have another order than the scan's, so the 32-bit mode keeps the scan.
#include "common.cuh"

#define LT_CH_MAX 16             // rows staged at a time by the scan (half as many for the largest heads: shared memory)
#define LT_COLS 16               // value columns of a scan block
#define LT_PARTS 16              // parts the key rows are cut in: a part is a half-warp, its rows lie side by side
#define LT_THREADS (LT_COLS * LT_PARTS)

template <int ACT> __device__ __forceinline__ float lt_act(float z) {
    return ACT == 0 ? z / (1.0f + expf(-z)) : z;
}

// One element of a rotated pair: `x` is the element itself, `y` its partner (i + rot/2 for the lower half, i - rot/2 for
// the upper); (u, v) -> (u c - v s, v c + u s).
__device__ __forceinline__ void lt_rotate(float& x, float y, float c, float s, bool lower) {
    x = lower ? x * c - y * s : x * c + y * s;
}

// R: key rows a thread keeps (dim <= LT_PARTS * R).  Thread (part p, column c) owns rows p R .. p R + R - 1 of column c.
template <typename T, int R, int ACT>
__global__ void __launch_bounds__(LT_THREADS)
lightning_scan_kernel(const T* __restrict__ qkv, int ld, int q_col, int k_col, int v_col, const float* __restrict__ decay_hi,
                      const float* __restrict__ decay_lo, float* __restrict__ state, const int* __restrict__ cu_rows,
                      const int* __restrict__ seg_pos, const int* __restrict__ seg_slot, float* __restrict__ o, int ldo, int H,
                      int dim, int vdim, int write_state, const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                      int rot, float k_scale) {
    kp_pdl_begin();
    constexpr int DP = LT_PARTS * R;                             // the key rows, padded with zeros
    constexpr int LT_CH = R >= 16 ? LT_CH_MAX / 2 : LT_CH_MAX;
    __shared__ __align__(16) float sq[LT_CH][DP];
    __shared__ __align__(16) float sk[LT_CH][DP];
    __shared__ float sv[LT_CH][LT_COLS];
    __shared__ float part[LT_CH][LT_PARTS][LT_COLS];
    const int seg = blockIdx.x, head = blockIdx.y, tile = blockIdx.z;
    const int c = threadIdx.x & (LT_COLS - 1), p = threadIdx.x / LT_COLS;
    const int j = tile * LT_COLS + c;
    const bool jok = j < vdim;
    const float ahi = decay_hi[head], alo = decay_lo[head];
    float* st = state + (((size_t)seg_slot[seg] * H + head) * dim) * vdim;
    float s[R];
    const bool fresh = seg_pos[seg] == 0;
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int i = p * R + r;
        s[r] = (!fresh && jok && i < dim) ? st[(size_t)i * vdim + j] : 0.f;
    }
    const int row0 = cu_rows[seg], row1 = cu_rows[seg + 1];
    for (int t0 = row0; t0 < row1; t0 += LT_CH) {
        const int nt = min(LT_CH, row1 - t0);
        __syncthreads();
        for (int x = threadIdx.x; x < nt * DP; x += LT_THREADS) {
            const int t = x / DP, i = x - t * DP;
            float qv = 0.f, kv = 0.f;
            if (i < dim) {
                const T* row = qkv + (size_t)(t0 + t) * ld + head * dim + i;
                qv = lt_act<ACT>(to_f32(row[q_col]));
                kv = lt_act<ACT>(to_f32(row[k_col]));
                if (i < rot) {
                    const int half = rot >> 1, lowr = i < half;
                    const T* prow = lowr ? row + half : row - half;
                    const size_t tb = (size_t)(seg_pos[seg] + (t0 + t - row0)) * half + (lowr ? i : i - half);
                    lt_rotate(qv, lt_act<ACT>(to_f32(prow[q_col])), cos_tab[tb], sin_tab[tb], lowr);
                    lt_rotate(kv, lt_act<ACT>(to_f32(prow[k_col])), cos_tab[tb], sin_tab[tb], lowr);
                }
                kv *= k_scale;
            }
            sq[t][i] = qv;
            sk[t][i] = kv;
        }
        for (int x = threadIdx.x; x < nt * LT_COLS; x += LT_THREADS) {
            const int t = x / LT_COLS, l = x % LT_COLS, jj = tile * LT_COLS + l;
            sv[t][l] = jj < vdim ? lt_act<ACT>(to_f32(qkv[(size_t)(t0 + t) * ld + v_col + head * vdim + jj])) : 0.f;
        }
        __syncthreads();
        for (int t = 0; t < nt; t++) {
            const float vj = sv[t][c];
            const float* kt = &sk[t][p * R];
            const float* qt = &sq[t][p * R];
            float acc = 0.f;
            if (R % 4 == 0) {
#pragma unroll
                for (int r = 0; r < R; r += 4) {
                    const float4 k4 = *reinterpret_cast<const float4*>(kt + r), q4 = *reinterpret_cast<const float4*>(qt + r);
                    s[r] = fmaf(ahi, s[r], fmaf(k4.x, vj, alo * s[r]));
                    acc = fmaf(s[r], q4.x, acc);
                    s[r + 1] = fmaf(ahi, s[r + 1], fmaf(k4.y, vj, alo * s[r + 1]));
                    acc = fmaf(s[r + 1], q4.y, acc);
                    s[r + 2] = fmaf(ahi, s[r + 2], fmaf(k4.z, vj, alo * s[r + 2]));
                    acc = fmaf(s[r + 2], q4.z, acc);
                    s[r + 3] = fmaf(ahi, s[r + 3], fmaf(k4.w, vj, alo * s[r + 3]));
                    acc = fmaf(s[r + 3], q4.w, acc);
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; r++) {
                    s[r] = fmaf(ahi, s[r], fmaf(kt[r], vj, alo * s[r]));
                    acc = fmaf(s[r], qt[r], acc);
                }
            }
            part[t][p][c] = acc;
        }
        __syncthreads();
        for (int x = threadIdx.x; x < nt * LT_COLS; x += LT_THREADS) {
            const int t = x / LT_COLS, l = x % LT_COLS, jj = tile * LT_COLS + l;
            float sum = part[t][0][l];
#pragma unroll
            for (int q = 1; q < LT_PARTS; q++) sum += part[t][q][l];
            if (jj < vdim) o[(size_t)(t0 + t) * ldo + head * vdim + jj] = sum;
        }
    }
    if (write_state && jok) {
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int i = p * R + r;
            if (i < dim) st[(size_t)i * vdim + j] = s[r];
        }
    }
}


// ------------------------------------------------------------------------------------------------ chunked
#define LC_C 64                  // rows of a chunk
#define LC_LD (LC_C + 4)         // row stride of the transposed q and k tiles and of P (banks: 4 r mod 32 for row r)
#define LC_COLS 32               // value columns of a block
#define LC_THREADS 256
#define LC_MAX_DIM 128

// ------------------------------------------------------------------------------------------ chunks in parallel
// The chunks of all segments side by side (a list built on the host: chunk -> segment, first row): (1) every chunk's own sum U_c = sum_j a^(n-1-j) k_j v_j^T, all chunks at once; (2) a short serial pass a
// (segment, head) turns the sums into the states at the chunks' heads, S_(c+1) = a^n S_c + U_c, in place, and leaves
// the segment's last state in its slot; (3) every chunk's outputs from its state and its own rows, all chunks at once.
// Only (2) is serial, and it is one multiply-add an element and chunk.

// A [rows t0 .. t0 + n) x [dim] stretch of columns, with the activation, transposed into dst [dim][LC_LD]
// (zeros behind the n rows).
// What staging needs to rotate and scale q or k: the tables, the rotated dimensions (0: none), the position of the
// chunk's first row and the constant factor.
struct LcRot { const float* cos_tab; const float* sin_tab; int rot; int pos0; float scale; };

template <typename T, int ACT, bool VEC>
__device__ __forceinline__ void lc_stage_transposed(float* dst, const T* __restrict__ qkv, int ld, int col, int head, int dim,
                                                    int t0, int n, int tid, const LcRot rp) {
    const int half = rp.rot >> 1;
    if (VEC && (half % 8 == 0)) {
        // an item is (row t, eight columns): a rotated pair of eights (columns g 8 .. and half + g 8 ..) is one item, so
        // that both halves and their cosines and sines are fetched once, 16 bytes a load
        const int ng = dim / 8, hg = half / 8;
        for (int x = tid; x < (ng - hg) * LC_C; x += LC_THREADS) {
            const int t = x % LC_C, j = x / LC_C;
            const bool pair = j < hg;
            const int g = pair ? j : j + hg;
            float lo8[8], hi8[8];
#pragma unroll
            for (int e = 0; e < 8; e++) lo8[e] = hi8[e] = 0.f;
            if (t < n) {
                const T* src = qkv + (size_t)(t0 + t) * ld + col + head * dim + g * 8;
                const uint4 raw = __ldg(reinterpret_cast<const uint4*>(src));
                const bf16* e8 = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
                for (int e = 0; e < 8; e++) lo8[e] = lt_act<ACT>(__bfloat162float(e8[e]));
                if (pair) {
                    const uint4 praw = __ldg(reinterpret_cast<const uint4*>(src + half));
                    const bf16* p8 = reinterpret_cast<const bf16*>(&praw);
                    const float4* ct = reinterpret_cast<const float4*>(rp.cos_tab + (size_t)(rp.pos0 + t) * half + g * 8);
                    const float4* st = reinterpret_cast<const float4*>(rp.sin_tab + (size_t)(rp.pos0 + t) * half + g * 8);
                    const float4 c0 = __ldg(ct), c1 = __ldg(ct + 1), s0 = __ldg(st), s1 = __ldg(st + 1);
                    const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const float u = lo8[e], w = lt_act<ACT>(__bfloat162float(p8[e]));
                        float a = u, b = w;
                        lt_rotate(a, w, cs[e], sn[e], true);
                        lt_rotate(b, u, cs[e], sn[e], false);
                        lo8[e] = a;
                        hi8[e] = b;
                    }
                }
            }
#pragma unroll
            for (int e = 0; e < 8; e++) {
                dst[(g * 8 + e) * LC_LD + t] = lo8[e] * rp.scale;
                if (pair) dst[(half + g * 8 + e) * LC_LD + t] = hi8[e] * rp.scale;
            }
        }
    } else {
        for (int x = tid; x < dim * LC_C; x += LC_THREADS) {
            const int t = x % LC_C, d = x / LC_C;
            float v = 0.f;
            if (t < n) {
                const T* src = qkv + (size_t)(t0 + t) * ld + col + head * dim + d;
                v = lt_act<ACT>(to_f32(*src));
                if (d < rp.rot) {
                    const bool lowr = d < half;
                    const size_t tb = (size_t)(rp.pos0 + t) * half + (lowr ? d : d - half);
                    lt_rotate(v, lt_act<ACT>(to_f32(lowr ? src[half] : src[-half])), rp.cos_tab[tb], rp.sin_tab[tb], lowr);
                }
            }
            dst[d * LC_LD + t] = v * rp.scale;
        }
    }
}

template <typename T, int ACT>
__device__ __forceinline__ void lc_stage_values(float* Vs, const T* __restrict__ qkv, int ld, int v_col, int head, int vdim,
                                                int tile, int t0, int n, int tid) {
    for (int x = tid; x < LC_C * LC_COLS; x += LC_THREADS) {
        const int t = x / LC_COLS, c = x % LC_COLS, j = tile * LC_COLS + c;
        Vs[x] = (t < n && j < vdim) ? lt_act<ACT>(to_f32(qkv[(size_t)(t0 + t) * ld + v_col + head * vdim + j])) : 0.f;
    }
}

// (1) U[chunk][head] = sum_j a^(n-1-j) k_j v_j^T
template <typename T, int ACT, bool VEC>
__global__ void __launch_bounds__(LC_THREADS)
lightning_chunk_sums_kernel(const T* __restrict__ qkv, int ld, int k_col, int v_col, const float* __restrict__ decay_pow,
                            const int* __restrict__ cu_rows, const int* __restrict__ chunk_seg,
                            const int* __restrict__ chunk_row0, float* __restrict__ U, int H, int dim, int vdim,
                            const int* __restrict__ seg_pos, const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                            int rot, float k_scale) {
    kp_pdl_begin();
    extern __shared__ __align__(16) float lc_sm[];
    float* Kt = lc_sm;                                           // [dim][LC_LD]
    float* Vs = Kt + (size_t)dim * LC_LD;                        // [LC_C][LC_COLS]
    float* kw = Vs + LC_C * LC_COLS;                             // [LC_C]
    const int chunk = blockIdx.x, head = blockIdx.y, tile = blockIdx.z, tid = threadIdx.x;
    const int t0 = chunk_row0[chunk], n = min(LC_C, cu_rows[chunk_seg[chunk] + 1] - t0);
    const int sg = chunk_seg[chunk];
    const LcRot rk = {cos_tab, sin_tab, rot, rot ? seg_pos[sg] + t0 - cu_rows[sg] : 0, k_scale};
    lc_stage_transposed<T, ACT, VEC>(Kt, qkv, ld, k_col, head, dim, t0, n, tid, rk);
    lc_stage_values<T, ACT>(Vs, qkv, ld, v_col, head, vdim, tile, t0, n, tid);
    for (int x = tid; x < LC_C; x += LC_THREADS) kw[x] = x < n ? decay_pow[(size_t)head * (LC_C + 1) + n - 1 - x] : 0.f;
    __syncthreads();
    const int r0 = (tid / 8) * 2, c0 = (tid % 8) * 4;
    float* Uc = U + ((size_t)chunk * H + head) * dim * vdim;
    for (int d0 = r0; d0 < dim; d0 += 2 * (LC_THREADS / 8)) {
        float acc[2][4];
#pragma unroll
        for (int a = 0; a < 2; a++)
#pragma unroll
            for (int b = 0; b < 4; b++) acc[a][b] = 0.f;
        const bool two = d0 + 1 < dim;
#pragma unroll 4
        for (int j = 0; j < n; j++) {
            const float w = kw[j];
            const float k0 = Kt[d0 * LC_LD + j] * w, k1 = two ? Kt[(d0 + 1) * LC_LD + j] * w : 0.f;
            const float4 v4 = *reinterpret_cast<const float4*>(Vs + j * LC_COLS + c0);
            acc[0][0] = fmaf(k0, v4.x, acc[0][0]); acc[0][1] = fmaf(k0, v4.y, acc[0][1]);
            acc[0][2] = fmaf(k0, v4.z, acc[0][2]); acc[0][3] = fmaf(k0, v4.w, acc[0][3]);
            acc[1][0] = fmaf(k1, v4.x, acc[1][0]); acc[1][1] = fmaf(k1, v4.y, acc[1][1]);
            acc[1][2] = fmaf(k1, v4.z, acc[1][2]); acc[1][3] = fmaf(k1, v4.w, acc[1][3]);
        }
#pragma unroll
        for (int a = 0; a < 2; a++) {
            if (d0 + a >= dim) continue;
#pragma unroll
            for (int b = 0; b < 4; b++) {
                const int j = tile * LC_COLS + c0 + b;
                if (j < vdim) Uc[(size_t)(d0 + a) * vdim + j] = acc[a][b];
            }
        }
    }
}

// (2) in place: U[chunk] <- the state at the chunk's head; the segment's slot <- the state behind its last chunk
__global__ void __launch_bounds__(256)
lightning_chunk_states_kernel(float* __restrict__ U, const float* __restrict__ decay_pow, float* __restrict__ state,
                              const int* __restrict__ cu_rows, const int* __restrict__ seg_pos, const int* __restrict__ seg_slot,
                              const int* __restrict__ seg_chunk0, const int* __restrict__ chunk_row0, int H, int dim, int vdim,
                              int write_state) {
    kp_pdl_begin();
    const int seg = blockIdx.x, head = blockIdx.y;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    if (e >= dim * vdim) return;
    float* st = state + (((size_t)seg_slot[seg] * H + head) * dim) * vdim + e;
    float S = seg_pos[seg] == 0 ? 0.f : *st;
    const int row1 = cu_rows[seg + 1];
    // (eight chunks' sums are fetched at once: the serial part is then the multiply-adds alone, not the loads' latency)
    const size_t stride = (size_t)H * dim * vdim;
    const int c_end = seg_chunk0[seg + 1];
    for (int c0 = seg_chunk0[seg]; c0 < c_end; c0 += 8) {
        float* p = U + ((size_t)c0 * H + head) * dim * vdim + e;
        float u[8];
        float w[8];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            if (c0 + k < c_end) {
                u[k] = p[k * stride];
                w[k] = decay_pow[(size_t)head * (LC_C + 1) + min(LC_C, row1 - chunk_row0[c0 + k])];
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

// (3) o_i = sum_{j <= i} a^(i-j) (q_i . k_j) v_j + a^(i+1) q_i^T S, S the state at the chunk's head
template <typename T, int ACT, bool VEC>
__global__ void __launch_bounds__(LC_THREADS)
lightning_chunk_out_kernel(const T* __restrict__ qkv, int ld, int q_col, int k_col, int v_col, const float* __restrict__ decay_pow,
                           const int* __restrict__ cu_rows, const int* __restrict__ chunk_seg, const int* __restrict__ chunk_row0,
                           const float* __restrict__ U, float* __restrict__ o, int ldo, int H, int dim, int vdim,
                           const int* __restrict__ seg_pos, const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                           int rot, float k_scale) {
    kp_pdl_begin();
    extern __shared__ __align__(16) float lc_sm[];
    float* Qt = lc_sm;                                           // [dim][LC_LD]
    float* Kt = Qt + (size_t)dim * LC_LD;                        // [dim][LC_LD]
    float* Vs = Kt + (size_t)dim * LC_LD;                        // [LC_C][LC_COLS]
    float* Ps = Vs + LC_C * LC_COLS;                             // [LC_C][LC_LD]
    float* Ss = Ps + LC_C * LC_LD;                               // [dim][LC_COLS]
    float* pw = Ss + (size_t)dim * LC_COLS;                      // [LC_C + 1]
    const int chunk = blockIdx.x, head = blockIdx.y, tile = blockIdx.z, tid = threadIdx.x;
    const int t0 = chunk_row0[chunk], n = min(LC_C, cu_rows[chunk_seg[chunk] + 1] - t0);
    const int sg = chunk_seg[chunk];
    const int pos0 = rot ? seg_pos[sg] + t0 - cu_rows[sg] : 0;
    const LcRot rq = {cos_tab, sin_tab, rot, pos0, 1.0f}, rk = {cos_tab, sin_tab, rot, pos0, k_scale};
    lc_stage_transposed<T, ACT, VEC>(Qt, qkv, ld, q_col, head, dim, t0, n, tid, rq);
    lc_stage_transposed<T, ACT, VEC>(Kt, qkv, ld, k_col, head, dim, t0, n, tid, rk);
    lc_stage_values<T, ACT>(Vs, qkv, ld, v_col, head, vdim, tile, t0, n, tid);
    const float* Sc = U + ((size_t)chunk * H + head) * dim * vdim;
    for (int x = tid; x < dim * LC_COLS; x += LC_THREADS) {
        const int d = x / LC_COLS, c = x % LC_COLS, j = tile * LC_COLS + c;
        Ss[x] = j < vdim ? Sc[(size_t)d * vdim + j] : 0.f;
    }
    for (int x = tid; x <= LC_C; x += LC_THREADS) pw[x] = decay_pow[(size_t)head * (LC_C + 1) + x];
    __syncthreads();
    const int i0 = (tid / 16) * 4, j0 = (tid % 16) * 4;
    const int r0 = (tid / 8) * 2, c0 = (tid % 8) * 4;
    {
        float acc[4][4];
#pragma unroll
        for (int a = 0; a < 4; a++)
#pragma unroll
            for (int b = 0; b < 4; b++) acc[a][b] = 0.f;
        if (j0 <= i0 + 3 && i0 < n) {
#pragma unroll 4
            for (int d = 0; d < dim; d++) {
                const float4 q4 = *reinterpret_cast<const float4*>(Qt + d * LC_LD + i0);
                const float4 k4 = *reinterpret_cast<const float4*>(Kt + d * LC_LD + j0);
                const float qa[4] = {q4.x, q4.y, q4.z, q4.w}, kb[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
                for (int a = 0; a < 4; a++)
#pragma unroll
                    for (int b = 0; b < 4; b++) acc[a][b] = fmaf(qa[a], kb[b], acc[a][b]);
            }
        }
#pragma unroll
        for (int a = 0; a < 4; a++) {
            float4 out;
            float* po = reinterpret_cast<float*>(&out);
#pragma unroll
            for (int b = 0; b < 4; b++) {
                const int i = i0 + a, j = j0 + b;
                po[b] = j <= i ? acc[a][b] * pw[i - j] : 0.f;
            }
            *reinterpret_cast<float4*>(Ps + (i0 + a) * LC_LD + j0) = out;
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
        const float p0 = Ps[r0 * LC_LD + j], p1 = Ps[(r0 + 1) * LC_LD + j];
        const float4 v4 = *reinterpret_cast<const float4*>(Vs + j * LC_COLS + c0);
        ap[0][0] = fmaf(p0, v4.x, ap[0][0]); ap[0][1] = fmaf(p0, v4.y, ap[0][1]);
        ap[0][2] = fmaf(p0, v4.z, ap[0][2]); ap[0][3] = fmaf(p0, v4.w, ap[0][3]);
        ap[1][0] = fmaf(p1, v4.x, ap[1][0]); ap[1][1] = fmaf(p1, v4.y, ap[1][1]);
        ap[1][2] = fmaf(p1, v4.z, ap[1][2]); ap[1][3] = fmaf(p1, v4.w, ap[1][3]);
    }
#pragma unroll 4
    for (int d = 0; d < dim; d++) {
        const float2 q2 = *reinterpret_cast<const float2*>(Qt + d * LC_LD + r0);
        const float4 s4 = *reinterpret_cast<const float4*>(Ss + d * LC_COLS + c0);
        as[0][0] = fmaf(q2.x, s4.x, as[0][0]); as[0][1] = fmaf(q2.x, s4.y, as[0][1]);
        as[0][2] = fmaf(q2.x, s4.z, as[0][2]); as[0][3] = fmaf(q2.x, s4.w, as[0][3]);
        as[1][0] = fmaf(q2.y, s4.x, as[1][0]); as[1][1] = fmaf(q2.y, s4.y, as[1][1]);
        as[1][2] = fmaf(q2.y, s4.z, as[1][2]); as[1][3] = fmaf(q2.y, s4.w, as[1][3]);
    }
#pragma unroll
    for (int a = 0; a < 2; a++) {
        const int i = r0 + a;
        if (i >= n) continue;
        const float w = pw[i + 1];
        float* dst = o + (size_t)(t0 + i) * ldo + head * vdim + tile * LC_COLS + c0;
#pragma unroll
        for (int b = 0; b < 4; b++)
            if (tile * LC_COLS + c0 + b < vdim) dst[b] = fmaf(w, as[a][b], ap[a][b]);
    }
}

extern "C" {

// qkv: rows [n, ld] in the storage type; q, k at columns q_col, k_col (H heads of dim), v at v_col (H heads of vdim).
// decay_hi + decay_lo: the heads' decays [H].  state: [slots, H, dim, vdim] float32.  o: [n, ldo] float32, heads side by
// side.  act: 0 silu on q, k and v; 1 none.  Segments as everywhere: cu_rows [n_seg + 1], seg_pos, seg_slot [n_seg].
// cos_tab, sin_tab [positions][rot / 2] and rot (even, at most dim; 0 and null tables: no rotation); k_scale: the factor
// on k behind the rotation (1 for none).
int kp_lightning_scan(const void* qkv, int ld, int q_col, int k_col, int v_col, const float* decay_hi, const float* decay_lo,
                      float* state, const int* cu_rows, const int* seg_pos, const int* seg_slot, float* o, int ldo, int n_seg,
                      int H, int dim, int vdim, int act, int write_state, const float* cos_tab, const float* sin_tab, int rot,
                      float k_scale, int dtype, void* stream) {
    if (n_seg <= 0) return 0;
    if (H < 1 || dim < 1 || vdim < 1 || act < 0 || act > 1) return KP_ERR_BAD_ARG;
    if (rot < 0 || (rot & 1) || rot > dim || (rot > 0 && (!cos_tab || !sin_tab))) return KP_ERR_BAD_ARG;
    if (dim > 16 * LT_PARTS || H > 65535 || (vdim + LT_COLS - 1) / LT_COLS > 65535) return KP_ERR_UNSUPPORTED;
    const dim3 grid(n_seg, H, (vdim + LT_COLS - 1) / LT_COLS), block(LT_THREADS);
    cudaStream_t s = (cudaStream_t)stream;
#define LT_LAUNCH(T, R, ACT)                                                                                                 \
    kp_launch_pdl(lightning_scan_kernel<T, R, ACT>, grid, block, 0, s, (const T*)qkv, ld, q_col, k_col, v_col, decay_hi, decay_lo, \
                  state, cu_rows, seg_pos, seg_slot, o, ldo, H, dim, vdim, write_state, cos_tab, sin_tab, rot, k_scale)
    // (the rows a thread keeps depend on the head's size only, so a row's sums have the same order in every launch)
#define LT_BY_R(T, ACT)                                                                                                      \
    do {                                                                                                                     \
        if (dim <= 2 * LT_PARTS) LT_LAUNCH(T, 2, ACT);                                                                       \
        else if (dim <= 4 * LT_PARTS) LT_LAUNCH(T, 4, ACT);                                                                  \
        else if (dim <= 8 * LT_PARTS) LT_LAUNCH(T, 8, ACT);                                                                  \
        else LT_LAUNCH(T, 16, ACT);                                                                                          \
    } while (0)
    KP_DISPATCH_DTYPE(dtype, T, { if (act == 0) LT_BY_R(T, 0); else LT_BY_R(T, 1); });
#undef LT_BY_R
#undef LT_LAUNCH
    return kp_launch_status();
}

// Rows of a chunk of the chunked form (the decay table holds a^0 .. a^rows for every head).
int kp_lightning_chunk_rows() { return LC_C; }

// The chunked form: the arguments of kp_lightning_scan with the decays given as powers, decay_pow [H][rows + 1] = a_h^m,
// and the list of chunks.  KP_ERR_UNSUPPORTED for heads it does not take (dim > 128).  chunk_seg, chunk_row0 [n_chunks]: every chunk's segment and first row
// (chunks of at most kp_lightning_chunk_rows() rows, a segment's chunks in order and side by side); seg_chunk0 [n_seg + 1]:
// the first chunk of every segment; scratch: n_chunks * H * dim * vdim floats.
int kp_lightning_chunks(const void* qkv, int ld, int q_col, int k_col, int v_col, const float* decay_pow, float* state,
                        const int* cu_rows, const int* seg_pos, const int* seg_slot, const int* chunk_seg, const int* chunk_row0,
                        const int* seg_chunk0, int n_chunks, float* scratch, float* o, int ldo, int n_seg, int H, int dim, int vdim,
                        int act, int write_state, const float* cos_tab, const float* sin_tab, int rot, float k_scale, int dtype,
                        void* stream) {
    if (n_seg <= 0 || n_chunks <= 0) return 0;
    if (H < 1 || dim < 1 || vdim < 1 || act < 0 || act > 1) return KP_ERR_BAD_ARG;
    if (rot < 0 || (rot & 1) || rot > dim || (rot > 0 && (!cos_tab || !sin_tab))) return KP_ERR_BAD_ARG;
    const int tiles = (vdim + LC_COLS - 1) / LC_COLS;
    if (dim > LC_MAX_DIM || H > 65535 || tiles > 65535 || (dim * vdim + 255) / 256 > 65535) return KP_ERR_UNSUPPORTED;
    const size_t sm1 = ((size_t)dim * LC_LD + LC_C * LC_COLS + LC_C) * sizeof(float);
    const size_t sm3 = ((size_t)2 * dim * LC_LD + LC_C * LC_COLS + LC_C * LC_LD + (size_t)dim * LC_COLS + LC_C + 4) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
#define LC3_LAUNCH(T, ACT, VEC)                                                                                              \
    do {                                                                                                                     \
        if ((e = cudaFuncSetAttribute(lightning_chunk_sums_kernel<T, ACT, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm1)) != cudaSuccess) return (int)e; \
        if ((e = cudaFuncSetAttribute(lightning_chunk_out_kernel<T, ACT, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm3)) != cudaSuccess) return (int)e; \
        kp_launch_pdl(lightning_chunk_sums_kernel<T, ACT, VEC>, dim3(n_chunks, H, tiles), dim3(LC_THREADS), sm1, s, (const T*)qkv, ld, \
                      k_col, v_col, decay_pow, cu_rows, chunk_seg, chunk_row0, scratch, H, dim, vdim, seg_pos, cos_tab, sin_tab, rot, k_scale);                      \
        if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;                                                          \
        kp_launch_pdl(lightning_chunk_states_kernel, dim3(n_seg, H, (dim * vdim + 255) / 256), dim3(256), 0, s, scratch, decay_pow, \
                      state, cu_rows, seg_pos, seg_slot, seg_chunk0, chunk_row0, H, dim, vdim, write_state);                 \
        if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;                                                          \
        kp_launch_pdl(lightning_chunk_out_kernel<T, ACT, VEC>, dim3(n_chunks, H, tiles), dim3(LC_THREADS), sm3, s, (const T*)qkv, ld, \
                      q_col, k_col, v_col, decay_pow, cu_rows, chunk_seg, chunk_row0, (const float*)scratch, o, ldo, H, dim, vdim, seg_pos, cos_tab, sin_tab, rot, k_scale); \
    } while (0)
    // (with a rotation whose half is a multiple of 8 the vector staging also fetches cosines and sines 16 bytes at a time)
    const bool tabs_ok = rot == 0 || (rot / 2) % 8 != 0 || (!((uintptr_t)cos_tab & 15) && !((uintptr_t)sin_tab & 15));
    const bool vec = dtype == KP_DTYPE_BF16 && dim % 8 == 0 && ld % 8 == 0 && q_col % 8 == 0 && k_col % 8 == 0 && !((uintptr_t)qkv & 15) && tabs_ok;
    if (vec) {
        if (act == 0) LC3_LAUNCH(bf16, 0, true); else LC3_LAUNCH(bf16, 1, true);
    } else {
        KP_DISPATCH_DTYPE(dtype, T, { if (act == 0) LC3_LAUNCH(T, 0, false); else LC3_LAUNCH(T, 1, false); });
    }
#undef LC3_LAUNCH
    return kp_launch_status();
}

}  // extern "C"
