// Mixture of experts: every row (token) runs `top` of E small gated feed-forward units and adds their
// outputs, weighted, to the float32 residual.
//
//   z = router logits [n, E] (float32, computed by the caller)
//   chosen(r) = the `top` largest z[r, :] (ties: the lower index), weights = softmax over the chosen logits only
//   out[r, :] += sum_j weight_j * Wd_e (act(Wg_e h_r) * (Wu_e h_r)),  e = chosen_j(r), j in order
//
// A second way of choosing (`mode` 1): scores s = softmax(z) over ALL router outputs; the `top` largest s + b are
// chosen (b: a correction that takes part in the choice only), and the weights are the chosen s themselves times a
// constant, not renormalised.  The last `n_identity` router outputs may stand for experts without weights that
// return their input: their pairs get places in the layout but no tiles, and the combine adds weight * h for them.
//
// A third (`mode` 2): the `top` largest logits are chosen, as in the first, and the weight of a chosen expert is
// sigmoid(z) times the constant, each on its own, not renormalised.
//
// The weight may multiply the expert's input instead of its output (`weight_input`): out[r, :] += sum_j unit_e(w_j h_r).
// The rows are then gathered place by place with their weights applied (float32 product, rounded to the storage
// type), the grouped products read the gathered rows, and the combine adds the outputs as they are.
//
// Which rows meet which expert is known on the device only, so the work is laid out there too and nothing
// comes back to the host (a step with this layer can be captured in a CUDA graph):
//   moe_route:  one warp a row picks the experts and their weights;
//   moe_sort:   one CTA counts the (row, choice) pairs of every expert, lays the pairs out expert by expert
//               (`perm`: place -> pair, `inv`: pair -> place) and lists the row tiles of every expert;
//   moe_gate_up / moe_down: grouped products over those tiles, a tile being rows of ONE expert, so that its
//               weights are read once for all of them; every output element sums k in order, whatever the
//               tile it fell into, so a row's result does not depend on the rest of the batch;
//   moe_combine: out[r] += sum over j of weight_j * y[place of (r, j)], j ascending.
// The products exist in two forms: CUDA-core float32 FMA (the true 32-bit path, and every shape), and
// bfloat16 tensor-core tiles (mma.sync m16n8k16, float32 accumulation) for 16-bit storage.
#include "tcgen05.cuh"

#define MOE_BM 32                // rows of a tile of the mma.sync and CUDA-core products
#define MOE_BIG 128              // rows of a tile of the tcgen05 products
#define MOE_MAX_TOP 32
#define MOE_SORT_THREADS 1024

// ------------------------------------------------------------------------------------------------ route
// One warp chooses for one row.  z [E]: the row's router logits in shared memory (mode 0: bias already added); they
// are overwritten.  s [E]: room for the scores of mode 1.
__device__ __forceinline__ void moe_choose(float* z, float* s, int E, int top, int mode, const float* __restrict__ bias,
                                           float wscale, int* __restrict__ idx_out, float* __restrict__ w_out) {
    const int lane = threadIdx.x & 31;
    if (mode == 1) {
        // scores over all outputs; the choice runs over score + correction, the weight is the score
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, z[e]);
        m = warp_max(m);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) { const float p = expf(z[e] - m); s[e] = p; sum += p; }
        sum = warp_sum(sum);
        for (int e = lane; e < E; e += 32) {
            const float sc = s[e] / sum;
            s[e] = sc;
            z[e] = sc + (bias ? bias[e] : 0.f);
        }
        __syncwarp();
    }
    float my_z = -INFINITY;
    int my_e = 0;
    for (int j = 0; j < top; j++) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (v > best) { best = v; bi = e; }                 // (ascending e: the first of equal values stays)
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (bi == 0x7fffffff) bi = 0;                           // (a row of NaN or -inf: keep the indices legal)
        if (lane == j) { my_z = best; my_e = bi; }
        if (lane == 0) z[bi] = -INFINITY;
        __syncwarp();
    }
    if (mode == 1) {
        if (lane < top) {
            idx_out[lane] = my_e;
            w_out[lane] = s[my_e] * wscale;
        }
        return;
    }
    if (mode == 2) {
        if (lane < top) {
            idx_out[lane] = my_e;
            w_out[lane] = wscale / (1.0f + expf(-my_z));
        }
        return;
    }
    const float m = __shfl_sync(0xffffffffu, my_z, 0);
    const float p = lane < top ? expf(my_z - m) : 0.f;
    const float sum = warp_sum(p);
    if (lane < top) {
        idx_out[lane] = my_e;
        w_out[lane] = p / sum;
    }
}

__global__ void __launch_bounds__(256)
moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int n, int E, int top, int mode,
                 float wscale, int* __restrict__ idx_out, float* __restrict__ w_out) {
    kp_pdl_begin();
    extern __shared__ float route_sm[];                         // [warps][2 E]: logits, scores
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = blockIdx.x * (blockDim.x >> 5) + warp;
    if (r >= n) return;
    float* z = route_sm + (size_t)warp * 2 * E;
    for (int e = lane; e < E; e += 32) z[e] = logits[(size_t)r * E + e] + (mode == 0 && bias ? bias[e] : 0.f);
    __syncwarp();
    moe_choose(z, z + E, E, top, mode, bias, wscale, idx_out + (size_t)r * top, w_out + (size_t)r * top);
}

// The router as one kernel: logits z = h Wr^T + b in float32 (h is widened from its storage type; a row's
// logit sums k in an order fixed by the lane pattern, whatever the batch), then the choice as above.  A block
// takes MOE_RB rows, which stay in shared memory as float32 while each warp walks its experts' rows of Wr.
// (RB rows a block: 8 for steps of many rows, so that Wr is fetched from L2 an eighth as often, 1 for steps of few,
// so that every row has a block of its own.  A warp takes four of its experts at a time: their loads are in
// flight together.  The order in which a (row, expert) logit adds up does not depend on RB.)
template <typename T, int RB>
__global__ void __launch_bounds__(256)
moe_router_kernel(const T* __restrict__ h, int ldh, const float* __restrict__ wr, const float* __restrict__ bias, int n,
                  int E, int d, int top, int mode, float wscale, int* __restrict__ idx_out, float* __restrict__ w_out) {
    kp_pdl_begin();
    extern __shared__ __align__(16) float router_sm[];          // [RB][d] rows, [RB][2 E] logits and scores
    float* hs = router_sm;
    float* zs = router_sm + (size_t)RB * d;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row0 = blockIdx.x * RB, nr = min(RB, n - row0);
    for (int i = threadIdx.x; i < RB * d; i += blockDim.x) {
        const int r = i / d, k = i - r * d;
        hs[i] = r < nr ? to_f32(h[(size_t)(row0 + r) * ldh + k]) : 0.f;
    }
    __syncthreads();
    for (int e0 = warp; e0 < E; e0 += 32) {                     // experts e0, e0 + 8, e0 + 16, e0 + 24 of this warp
        const float4* w4[4];
        bool has[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            has[j] = e0 + 8 * j < E;
            w4[j] = reinterpret_cast<const float4*>(wr + (size_t)(has[j] ? e0 + 8 * j : e0) * d);
        }
        float acc[4][RB];
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int r = 0; r < RB; r++) acc[j][r] = 0.f;
        for (int k = lane * 4; k < d; k += 128) {
            float4 w[4];
#pragma unroll
            for (int j = 0; j < 4; j++) w[j] = __ldg(w4[j] + (k >> 2));
#pragma unroll
            for (int r = 0; r < RB; r++) {
                const float4 x = *reinterpret_cast<const float4*>(hs + (size_t)r * d + k);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    acc[j][r] = fmaf(x.x, w[j].x, acc[j][r]); acc[j][r] = fmaf(x.y, w[j].y, acc[j][r]);
                    acc[j][r] = fmaf(x.z, w[j].z, acc[j][r]); acc[j][r] = fmaf(x.w, w[j].w, acc[j][r]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int r = 0; r < RB; r++) {
                const float v = warp_sum(acc[j][r]);
                if (lane == 0 && has[j]) zs[(size_t)r * 2 * E + e0 + 8 * j] = v + (mode == 0 && bias ? bias[e0 + 8 * j] : 0.f);
            }
    }
    __syncthreads();
    if (warp >= nr) return;
    float* z = zs + (size_t)warp * 2 * E;                        // warp r chooses for row r
    moe_choose(z, z + E, E, top, mode, bias, wscale, idx_out + (size_t)(row0 + warp) * top, w_out + (size_t)(row0 + warp) * top);
}

// ------------------------------------------------------------------------------------------------- sort
// offsets[e] .. offsets[e+1]: the places of expert e's pairs; tile_start[e] .. tile_start[e+1]: its row tiles
// of MOE_BM places (tile_start[E] = all tiles), big_start the same for tiles of MOE_BIG places.
// perm[place] = pair (row * top + j); inv[pair] = place.
__global__ void __launch_bounds__(MOE_SORT_THREADS)
moe_sort_kernel(const int* __restrict__ idx, int n_pairs, int E, int E_real, int* __restrict__ offsets, int* __restrict__ tile_start,
                int* __restrict__ big_start, int* __restrict__ perm, int* __restrict__ inv) {
    kp_pdl_begin();
    extern __shared__ int sort_sm[];                            // [E] counts, [E] cursors, [E + 1] offsets
    int* cnt = sort_sm;
    int* cur = cnt + E;
    int* off = cur + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) { cnt[e] = 0; cur[e] = 0; }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&cnt[idx[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int o = 0, t = 0, tb = 0;
        for (int e = 0; e < E; e++) {
            off[e] = o; offsets[e] = o; tile_start[e] = t; big_start[e] = tb;
            o += cnt[e];
            if (e < E_real) {                                   // (experts without weights have places but no tiles)
                t += (cnt[e] + MOE_BM - 1) / MOE_BM;
                tb += (cnt[e] + MOE_BIG - 1) / MOE_BIG;
            }
        }
        off[E] = o; offsets[E] = o; tile_start[E] = t; big_start[E] = tb;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = idx[p];
        const int place = off[e] + atomicAdd(&cur[e], 1);
        perm[place] = p;
        inv[p] = place;
    }
}

// The expert and the rows of row tile `bt` (false: no such tile in this step).
__device__ __forceinline__ bool moe_tile(const int* __restrict__ offsets, const int* __restrict__ tile_start, int E, int bt,
                                         int& e, int& row0, int& row1, int rows_a_tile = MOE_BM) {
    if (bt >= tile_start[E]) return false;
    int lo = 0, hi = E;                                         // the last e with tile_start[e] <= bt
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (tile_start[mid] <= bt) lo = mid; else hi = mid;
    }
    e = lo;
    row0 = offsets[e] + (bt - tile_start[e]) * rows_a_tile;
    row1 = min(row0 + rows_a_tile, offsets[e + 1]);
    return true;
}

// ---------------------------------------------------------------------------- products on the CUDA cores
// act[place, c] = f(h_row . Wg_e[c]) * (h_row . Wu_e[c]); gate and up are rounded to the storage type before f,
// as the dense gated unit does.  w_gu: [E][2 ff][d], gate rows then up rows.
template <typename T>
__global__ void __launch_bounds__(256)
moe_gate_up_kernel(const T* __restrict__ h, int ldh, const T* __restrict__ w_gu, const int* __restrict__ offsets,
                   const int* __restrict__ tile_start, const int* __restrict__ perm, T* __restrict__ act, int E, int top,
                   int d, int ff, int act_kind) {
    kp_pdl_begin();
    constexpr int BN = 32, BK = 16;
    __shared__ float As[BK][MOE_BM + 1], Gs[BK][BN + 1], Us[BK][BN + 1];
    __shared__ int src_row[MOE_BM];
    int e, row0, row1;
    if (!moe_tile(offsets, tile_start, E, blockIdx.y, e, row0, row1)) return;
    const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
    const int n0 = blockIdx.x * BN;
    if (tid < MOE_BM) src_row[tid] = row0 + tid < row1 ? (perm ? perm[row0 + tid] / top : row0 + tid) : -1;
    __syncthreads();
    const T* wg = w_gu + (size_t)e * 2 * ff * d;
    const T* wu = wg + (size_t)ff * d;
    float ag[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, au[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    for (int k0 = 0; k0 < d; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int el = tid + i * 256, r = el / BK, c = el % BK, gk = k0 + c;
            const int sr = src_row[r];
            As[c][r] = (sr >= 0 && gk < d) ? to_f32(h[(size_t)sr * ldh + gk]) : 0.f;
            const bool ok = n0 + r < ff && gk < d;
            Gs[c][r] = ok ? to_f32(wg[(size_t)(n0 + r) * d + gk]) : 0.f;
            Us[c][r] = ok ? to_f32(wu[(size_t)(n0 + r) * d + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; k++) {
            const float a0 = As[k][ty * 2], a1 = As[k][ty * 2 + 1];
            const float g0 = Gs[k][tx * 2], g1 = Gs[k][tx * 2 + 1], u0 = Us[k][tx * 2], u1 = Us[k][tx * 2 + 1];
            ag[0][0] = fmaf(a0, g0, ag[0][0]); ag[0][1] = fmaf(a0, g1, ag[0][1]);
            ag[1][0] = fmaf(a1, g0, ag[1][0]); ag[1][1] = fmaf(a1, g1, ag[1][1]);
            au[0][0] = fmaf(a0, u0, au[0][0]); au[0][1] = fmaf(a0, u1, au[0][1]);
            au[1][0] = fmaf(a1, u0, au[1][0]); au[1][1] = fmaf(a1, u1, au[1][1]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int place = row0 + ty * 2 + i;
        if (place >= row1) continue;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int c = n0 + tx * 2 + j;
            if (c >= ff) continue;
            const float g = to_f32(from_f32<T>(ag[i][j])), u = to_f32(from_f32<T>(au[i][j]));
            act[(size_t)place * ff + c] = from_f32<T>(kp_act_rt(act_kind, g) * u);
        }
    }
}

// y[place, c] = act[place, :] . Wd_e[c, :]   (float32 out).  w_down: [E][d][ff].
template <typename T>
__global__ void __launch_bounds__(256)
moe_down_kernel(const T* __restrict__ act, const T* __restrict__ w_down, const int* __restrict__ offsets,
                const int* __restrict__ tile_start, float* __restrict__ y, int E, int d, int ff) {
    kp_pdl_begin();
    constexpr int BN = 64, BK = 16;
    __shared__ float As[BK][MOE_BM + 1], Ws[BK][BN + 1];
    int e, row0, row1;
    if (!moe_tile(offsets, tile_start, E, blockIdx.y, e, row0, row1)) return;
    const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
    const int n0 = blockIdx.x * BN;
    const T* wd = w_down + (size_t)e * d * ff;
    float acc[2][4];
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < ff; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int el = tid + i * 256, r = el / BK, c = el % BK, gk = k0 + c;
            As[c][r] = (row0 + r < row1 && gk < ff) ? to_f32(act[(size_t)(row0 + r) * ff + gk]) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int el = tid + i * 256, r = el / BK, c = el % BK, gk = k0 + c;
            Ws[c][r] = (n0 + r < d && gk < ff) ? to_f32(wd[(size_t)(n0 + r) * ff + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; k++) {
            const float a0 = As[k][ty * 2], a1 = As[k][ty * 2 + 1];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float w = Ws[k][tx * 4 + j];
                acc[0][j] = fmaf(a0, w, acc[0][j]);
                acc[1][j] = fmaf(a1, w, acc[1][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int place = row0 + ty * 2 + i;
        if (place >= row1) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int c = n0 + tx * 4 + j;
            if (c < d) y[(size_t)place * d + c] = acc[i][j];
        }
    }
}

// ------------------------------------------------------------------------ products on the tensor cores
// The same two products for bfloat16 with mma.sync m16n8k16 (float32 accumulation): a CTA of four warps
// takes one row tile of 32 places and 64 output columns; warp w owns columns 16 w .. 16 w + 15 (two n-tiles)
// of both 16-row halves.  Operands go through shared memory in k-blocks of 64 (rows padded to 72 halves: the
// fragment loads of a warp then fall into different banks).  Needs K % 8 == 0 (16-byte loads).
#define MOE_TC_BN 64
#define MOE_TC_BK 64
#define MOE_TC_LD 72

__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, const uint32_t* b) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// One k-block of an operand matrix of ROWS rows: first from global memory into registers (16 bytes a thread and
// turn; rows beyond `valid`, or with a negative source row, and columns beyond K are zero), later from the
// registers into shared memory.  Between the two the products of the block before run, so that the loads'
// latency passes under them (a CTA of a decode step has a handful of rows and lives on that latency).
template <int ROWS>
struct MoeFrag { uint4 v[ROWS * (MOE_TC_BK / 8) / 128]; };

template <int ROWS>
__device__ __forceinline__ void moe_tc_fetch(MoeFrag<ROWS>& f, const bf16* src, const int* src_rows, long long ld,
                                             int first_row, int valid, int k0, int K) {
#pragma unroll
    for (int i = 0; i < ROWS * (MOE_TC_BK / 8) / 128; i++) {
        const int el = threadIdx.x + i * 128;
        const int r = el / (MOE_TC_BK / 8), c8 = (el % (MOE_TC_BK / 8)) * 8;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        const long long sr = src_rows ? (long long)src_rows[r] : (r < valid ? (long long)first_row + r : -1);
        if (sr >= 0 && k0 + c8 < K) v = *reinterpret_cast<const uint4*>(src + sr * ld + k0 + c8);
        f.v[i] = v;
    }
}
template <int ROWS>
__device__ __forceinline__ void moe_tc_put(bf16 (*dst)[MOE_TC_LD], const MoeFrag<ROWS>& f) {
#pragma unroll
    for (int i = 0; i < ROWS * (MOE_TC_BK / 8) / 128; i++) {
        const int el = threadIdx.x + i * 128;
        *reinterpret_cast<uint4*>(&dst[el / (MOE_TC_BK / 8)][(el % (MOE_TC_BK / 8)) * 8]) = f.v[i];
    }
}

// acc[half][nt][4] += A[32 x BK] * W[warp's 16 columns x BK]^T for one staged k-block
__device__ __forceinline__ void moe_tc_block(float (*acc)[2][4], const bf16 (*As)[MOE_TC_LD], const bf16 (*Ws)[MOE_TC_LD],
                                             int warp, int lane) {
    const int gid = lane >> 2, tig = lane & 3;
#pragma unroll
    for (int kk = 0; kk < MOE_TC_BK; kk += 16) {
        uint32_t b[2][2];
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
            const bf16* wr = &Ws[warp * 16 + nt * 8 + gid][kk + tig * 2];
            b[nt][0] = *reinterpret_cast<const uint32_t*>(wr);
            b[nt][1] = *reinterpret_cast<const uint32_t*>(wr + 8);
        }
#pragma unroll
        for (int half = 0; half < 2; half++) {
            uint32_t a[4];
            const bf16* ar0 = &As[half * 16 + gid][kk + tig * 2];
            const bf16* ar1 = &As[half * 16 + gid + 8][kk + tig * 2];
            a[0] = *reinterpret_cast<const uint32_t*>(ar0);
            a[1] = *reinterpret_cast<const uint32_t*>(ar1);
            a[2] = *reinterpret_cast<const uint32_t*>(ar0 + 8);
            a[3] = *reinterpret_cast<const uint32_t*>(ar1 + 8);
#pragma unroll
            for (int nt = 0; nt < 2; nt++) mma_bf16_16816(acc[half][nt], a, b[nt]);
        }
    }
}

__global__ void __launch_bounds__(128)
moe_gate_up_tc_kernel(const bf16* __restrict__ h, int ldh, const bf16* __restrict__ w_gu, const int* __restrict__ offsets,
                      const int* __restrict__ tile_start, const int* __restrict__ perm, bf16* __restrict__ act, int E,
                      int top, int d, int ff, int act_kind) {
    kp_pdl_begin();
    __shared__ __align__(16) bf16 As[MOE_BM][MOE_TC_LD], Gs[MOE_TC_BN][MOE_TC_LD], Us[MOE_TC_BN][MOE_TC_LD];
    __shared__ int src_row[MOE_BM];
    int e, row0, row1;
    if (!moe_tile(offsets, tile_start, E, blockIdx.y, e, row0, row1)) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * MOE_TC_BN;
    if (tid < MOE_BM) src_row[tid] = row0 + tid < row1 ? (perm ? perm[row0 + tid] / top : row0 + tid) : -1;
    __syncthreads();
    const bf16* wg = w_gu + (size_t)e * 2 * ff * d;
    const bf16* wu = wg + (size_t)ff * d;
    const int w_valid = min(MOE_TC_BN, ff - n0);
    float ag[2][2][4] = {}, au[2][2][4] = {};
    MoeFrag<MOE_BM> fa;
    MoeFrag<MOE_TC_BN> fg, fu;
    moe_tc_fetch(fa, h, src_row, ldh, 0, 0, 0, d);
    moe_tc_fetch(fg, wg, nullptr, d, n0, w_valid, 0, d);
    moe_tc_fetch(fu, wu, nullptr, d, n0, w_valid, 0, d);
    for (int k0 = 0; k0 < d; k0 += MOE_TC_BK) {
        moe_tc_put(As, fa);
        moe_tc_put(Gs, fg);
        moe_tc_put(Us, fu);
        __syncthreads();
        if (k0 + MOE_TC_BK < d) {                    // the next block is on its way while this one is multiplied
            moe_tc_fetch(fa, h, src_row, ldh, 0, 0, k0 + MOE_TC_BK, d);
            moe_tc_fetch(fg, wg, nullptr, d, n0, w_valid, k0 + MOE_TC_BK, d);
            moe_tc_fetch(fu, wu, nullptr, d, n0, w_valid, k0 + MOE_TC_BK, d);
        }
        moe_tc_block(ag, As, Gs, warp, lane);
        moe_tc_block(au, As, Us, warp, lane);
        __syncthreads();
    }
    const int gid = lane >> 2, tig = lane & 3;
#pragma unroll
    for (int half = 0; half < 2; half++)
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int place = row0 + half * 16 + gid + (i >> 1) * 8;
                const int c = n0 + warp * 16 + nt * 8 + tig * 2 + (i & 1);
                if (place < row1 && c < ff) {
                    const float g = to_f32(__float2bfloat16_rn(ag[half][nt][i])), u = to_f32(__float2bfloat16_rn(au[half][nt][i]));
                    act[(size_t)place * ff + c] = __float2bfloat16_rn(kp_act_rt(act_kind, g) * u);
                }
            }
}

__global__ void __launch_bounds__(128)
moe_down_tc_kernel(const bf16* __restrict__ act, const bf16* __restrict__ w_down, const int* __restrict__ offsets,
                   const int* __restrict__ tile_start, float* __restrict__ y, int E, int d, int ff) {
    kp_pdl_begin();
    __shared__ __align__(16) bf16 As[MOE_BM][MOE_TC_LD], Ws[MOE_TC_BN][MOE_TC_LD];
    int e, row0, row1;
    if (!moe_tile(offsets, tile_start, E, blockIdx.y, e, row0, row1)) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * MOE_TC_BN;
    const bf16* wd = w_down + (size_t)e * d * ff;
    const int w_valid = min(MOE_TC_BN, d - n0);
    float acc[2][2][4] = {};
    MoeFrag<MOE_BM> fa;
    MoeFrag<MOE_TC_BN> fw;
    moe_tc_fetch(fa, act, nullptr, ff, row0, row1 - row0, 0, ff);
    moe_tc_fetch(fw, wd, nullptr, ff, n0, w_valid, 0, ff);
    for (int k0 = 0; k0 < ff; k0 += MOE_TC_BK) {
        moe_tc_put(As, fa);
        moe_tc_put(Ws, fw);
        __syncthreads();
        if (k0 + MOE_TC_BK < ff) {
            moe_tc_fetch(fa, act, nullptr, ff, row0, row1 - row0, k0 + MOE_TC_BK, ff);
            moe_tc_fetch(fw, wd, nullptr, ff, n0, w_valid, k0 + MOE_TC_BK, ff);
        }
        moe_tc_block(acc, As, Ws, warp, lane);
        __syncthreads();
    }
    const int gid = lane >> 2, tig = lane & 3;
#pragma unroll
    for (int half = 0; half < 2; half++)
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int place = row0 + half * 16 + gid + (i >> 1) * 8;
                const int c = n0 + warp * 16 + nt * 8 + tig * 2 + (i & 1);
                if (place < row1 && c < d) y[(size_t)place * d + c] = acc[half][nt][i];
            }
}

// --------------------------------------------------------------------- products on tcgen05 (many rows)
// The grouped products of a prompt portion on the 5th-generation tensor cores.  A CTA computes one tile:
// MOE_BIG places of one expert by 128 accumulator columns.  Warp 0 is the TMA producer (k-blocks of 64 through a
// ring of MT_STAGES stages: a box of 128 rows of the left operand, which lies place by place, and the expert's
// rows of W, both with the 128-byte swizzle), one lane of warp 1 issues the tcgen05.mma (128 x 128 x 16, the
// accumulator in tensor memory), warps 2 to 5 read the accumulator with tcgen05.ld, each its quarter of the
// lanes, and write the rows that belong to the expert (a box may reach into the next expert's places; what the
// MMA makes of those rows is not stored).  Gated form: the W tile is 64 gate rows and the matching 64 up rows,
// accumulator columns c and 64 + c are gate and up of output column c, and the epilogue writes
// act(gate) * up in bfloat16.  Plain form: 128 output columns in float32.  Two CTAs fit an SM, so one's
// epilogue runs under the other's main loop.  Every wait is bounded; one that gives up sets the status word.
KP_STATUS_WORD(g_moe_tc_status, moe_tc)

#define MT_BN 128
#define MT_BK 64
#define MT_STAGES 3
#define MT_THREADS 192
#define MT_A_BYTES (MOE_BIG * MT_BK * 2)
#define MT_B_BYTES (MT_BN * MT_BK * 2)

struct MtArgs {
    const int* offsets; const int* big_start;
    int E, K;
    int n_out;                 // output columns: ff (gated) or d
    int w_rows;                // rows of W an expert has: 2 ff (gated) or d
    int up_off;                // gated: the up rows lie this many rows behind the gate rows (ff)
    void* out; int ldo;
    int act;
};

template <bool GATED>
__global__ void __launch_bounds__(MT_THREADS)
moe_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, const MtArgs p) {
    constexpr int N_TILE = GATED ? MT_BN / 2 : MT_BN;
    extern __shared__ unsigned char mt_smem[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)mt_smem + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + (size_t)MT_STAGES * (MT_A_BYTES + MT_B_BYTES));
    uint64_t* empty = full + MT_STAGES;
    uint64_t* acc_full = empty + MT_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmA)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmW)) : "memory");
        for (int s = 0; s < MT_STAGES; s++) { kp_mbar_init(&full[s], 1); kp_mbar_init(&empty[s], 1); }
        kp_mbar_init(acc_full, 1);
        *abort_flag = 0;
        kp_mbar_init_fence();
    }
    if (warp == 1) kp_tmem_alloc(tmem_slot, MT_BN);
    kp_tc_fence_before();
    __syncthreads();
    kp_tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    kp_pdl_begin();                                  // the layout and the operands come from the kernels before

    int e = 0, row0 = 0, row1 = 0;
    const bool live = moe_tile(p.offsets, p.big_start, p.E, blockIdx.y, e, row0, row1, MOE_BIG);
    const int n0 = blockIdx.x * N_TILE;
    const int n_kb = (p.K + MT_BK - 1) / MT_BK;
    if (live && warp == 0) {
        if (lane == 0) {
            const int w0 = e * p.w_rows + n0;
            int s = 0;
            uint32_t ph = 0;
            for (int kb = 0; kb < n_kb; kb++) {
                if (*abort_flag || !kp_mbar_wait_bounded(&empty[s], ph ^ 1)) { *abort_flag = 1; break; }
                unsigned char* a_dst = tiles + (size_t)s * (MT_A_BYTES + MT_B_BYTES);
                kp_mbar_expect_tx(&full[s], MT_A_BYTES + MT_B_BYTES);
                kp_tma_load_2d(a_dst, &tmA, kb * MT_BK, row0, &full[s]);
                if (GATED) {
                    kp_tma_load_2d(a_dst + MT_A_BYTES, &tmW, kb * MT_BK, w0, &full[s]);
                    kp_tma_load_2d(a_dst + MT_A_BYTES + MT_B_BYTES / 2, &tmW, kb * MT_BK, w0 + p.up_off, &full[s]);
                } else {
                    kp_tma_load_2d(a_dst + MT_A_BYTES, &tmW, kb * MT_BK, w0, &full[s]);
                }
                if (++s == MT_STAGES) { s = 0; ph ^= 1; }
            }
        }
    } else if (live && warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = kp_umma_idesc(MOE_BIG, MT_BN);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int kb = 0; kb < n_kb; kb++) {
                if (*abort_flag || !kp_mbar_wait_bounded(&full[s], ph)) { *abort_flag = 1; ok = false; break; }
                kp_tc_fence_after();
                const uint32_t a_addr = kp_smem_u32(tiles + (size_t)s * (MT_A_BYTES + MT_B_BYTES));
                const uint64_t adesc = kp_umma_desc(a_addr), bdesc = kp_umma_desc(a_addr + MT_A_BYTES);
#pragma unroll
                for (int k = 0; k < MT_BK / 16; k++) kp_umma_bf16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) ? 1u : 0u);
                kp_umma_commit(&empty[s]);
                if (++s == MT_STAGES) { s = 0; ph ^= 1; }
            }
            if (ok) kp_umma_commit(acc_full);
        }
    } else if (live) {
        const int q = warp & 3;                              // the quarter of the lanes this warp may read
        const bool ok = kp_mbar_wait_bounded(acc_full, 0) && !*abort_flag;
        if (!ok) *abort_flag = 1;
        kp_tc_fence_after();
        const int m = row0 + q * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
        if (ok) {
            if (GATED) {
                bf16* dst = (bf16*)p.out + (size_t)m * p.ldo;
                const bool vec = (p.ldo & 7) == 0 && (((uintptr_t)p.out) & 15) == 0;
#pragma unroll 1
                for (int c = 0; c < N_TILE; c += 32) {
                    uint32_t g[32], u[32];
                    kp_tmem_ld32_issue(lane_base + c, g);
                    kp_tmem_ld32_issue(lane_base + N_TILE + c, u);
                    kp_tmem_ld_wait();
                    if (m < row1) {
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const float gq = to_f32(from_f32<bf16>(__uint_as_float(g[j]))), uq = to_f32(from_f32<bf16>(__uint_as_float(u[j])));
                            v[j] = kp_act_rt(p.act, gq) * uq;
                        }
                        if (vec && n0 + c + 32 <= p.n_out) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                uint4 o;
                                __nv_bfloat162 t0 = __floats2bfloat162_rn(v[j], v[j + 1]), t1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                                __nv_bfloat162 t2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), t3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                                o.x = *reinterpret_cast<uint32_t*>(&t0); o.y = *reinterpret_cast<uint32_t*>(&t1);
                                o.z = *reinterpret_cast<uint32_t*>(&t2); o.w = *reinterpret_cast<uint32_t*>(&t3);
                                *reinterpret_cast<uint4*>(dst + n0 + c + j) = o;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (n0 + c + j < p.n_out) dst[n0 + c + j] = from_f32<bf16>(v[j]);
                        }
                    }
                }
            } else {
                float* dst = (float*)p.out + (size_t)m * p.ldo;
                const bool vec = (p.ldo & 3) == 0 && (((uintptr_t)p.out) & 15) == 0;
#pragma unroll 1
                for (int c = 0; c < N_TILE; c += 32) {
                    uint32_t r[32];
                    kp_tmem_ld32(lane_base + c, r);
                    if (m < row1) {
                        if (vec && n0 + c + 32 <= p.n_out) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                *reinterpret_cast<float4*>(dst + n0 + c + j) =
                                    make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (n0 + c + j < p.n_out) dst[n0 + c + j] = __uint_as_float(r[j]);
                        }
                    }
                }
            }
        }
    }
    kp_tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicExch(&g_moe_tc_status, 1);
        kp_linger_after_failure();
    }
    if (warp == 1) kp_tmem_dealloc(tmem_base, MT_BN);
}

// hs[place, :] = h[row of the pair at that place, :]   (16 bytes a thread and turn)
__global__ void moe_gather_rows_kernel(const bf16* __restrict__ h, int ldh, const int* __restrict__ perm, bf16* __restrict__ hs,
                                       int n_pairs, int d8, int top) {
    kp_pdl_begin();
    const size_t total = (size_t)n_pairs * d8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t place = i / d8, c = (i % d8) * 8;
        *reinterpret_cast<uint4*>(hs + place * (size_t)d8 * 8 + c) =
            *reinterpret_cast<const uint4*>(h + (size_t)(perm[place] / top) * ldh + c);
    }
}

// hs[place, :] = weight of the pair at that place * h[its row, :], the product in float32, rounded to the storage type.
template <typename T>
__global__ void moe_gather_scaled_kernel(const T* __restrict__ h, int ldh, const int* __restrict__ perm, const float* __restrict__ w,
                                         T* __restrict__ hs, int n_pairs, int d, int top) {
    kp_pdl_begin();
    const size_t total = (size_t)n_pairs * d;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t place = i / d, c = i % d;
        const int pair = perm[place];
        hs[i] = from_f32<T>(w[pair] * to_f32(h[(size_t)(pair / top) * ldh + c]));
    }
}
// The same for bfloat16 rows of a multiple of 8 columns that start on 16 bytes: 16 bytes a thread and turn.
__global__ void moe_gather_scaled_vec_kernel(const bf16* __restrict__ h, int ldh, const int* __restrict__ perm,
                                             const float* __restrict__ w, bf16* __restrict__ hs, int n_pairs, int d8, int top) {
    kp_pdl_begin();
    const size_t total = (size_t)n_pairs * d8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t place = i / d8, c = (i % d8) * 8;
        const int pair = perm[place];
        const float wt = w[pair];
        uint4 v = *reinterpret_cast<const uint4*>(h + (size_t)(pair / top) * ldh + c);
        __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 f = __bfloat1622float2(p2[j]);
            p2[j] = __floats2bfloat162_rn(wt * f.x, wt * f.y);
        }
        *reinterpret_cast<uint4*>(hs + place * (size_t)d8 * 8 + c) = v;
    }
}

// ---------------------------------------------------------------------------------------------- combine
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ inv, const float* __restrict__ w,
                                   float* __restrict__ out, int n, int d, int top) {
    kp_pdl_begin();
    const size_t total = (size_t)n * d;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / d, c = i % d;
        float s = 0.f;
        for (int j = 0; j < top; j++) s = fmaf(w ? w[r * top + j] : 1.f, y[(size_t)inv[r * top + j] * d + c], s);   // (no weights: they were applied to the inputs)
        out[i] += s;
    }
}

// The same where the experts from `E_real` on return their input: such a pair adds weight * h[r].
template <typename T>
__global__ void moe_combine_identity_kernel(const float* __restrict__ y, const int* __restrict__ inv, const float* __restrict__ w,
                                            const int* __restrict__ idx, const T* __restrict__ h, int ldh, int E_real,
                                            float* __restrict__ out, int n, int d, int top) {
    kp_pdl_begin();
    const size_t total = (size_t)n * d;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / d, c = i % d;
        float s = 0.f;
        for (int j = 0; j < top; j++) {
            const float v = idx[r * top + j] >= E_real ? to_f32(h[r * ldh + c]) : y[(size_t)inv[r * top + j] * d + c];
            s = fmaf(w[r * top + j], v, s);
        }
        out[i] += s;
    }
}

static long long g_moe_tc_min_pairs = 512;      // (row, choice) pairs from which the tcgen05 tiles are taken

extern "C" {

// For measurements and tests: the number of pairs from which the tcgen05 path runs.
void kp_moe_set_tc_min_pairs(long long v) { g_moe_tc_min_pairs = v; }

// Ints of scratch for the layout of one step: offsets, tile_start, big_start [E + 1 each], perm [n top], inv [n top].
long long kp_moe_layout_ints(int n, int E, int top) { return 3LL * (E + 1) + 2LL * n * top; }

// Row tiles a step of n rows can have at most (a grid axis of the grouped products).
int kp_moe_max_tiles(int n, int E, int top) {
    const long long pairs = (long long)n * top;
    return (int)(pairs / MOE_BM + (pairs < E ? pairs : E));
}

// logits [n, E] float32 -> idx [n, top], weights [n, top], and the layout (see kp_moe_layout_ints).
// mode 0: the largest logits (+ bias), weights = softmax over the chosen; mode 1: scores = softmax over all, the largest
// score + bias chosen, weights = score * wscale; mode 2: the largest logits, weights = sigmoid(logit) * wscale.  The last n_identity of the E outputs are experts without weights.
int kp_moe_route(const float* logits, const float* bias, int n, int E, int top, int mode, float wscale, int n_identity,
                 int* idx, float* weights, int* layout, void* stream) {
    if (n <= 0) return 0;
    if (E < 1 || top < 1 || top > E || top > MOE_MAX_TOP || mode < 0 || mode > 2 || n_identity < 0 || n_identity >= E)
        return KP_ERR_UNSUPPORTED;
    const size_t route_sm = (size_t)8 * 2 * E * sizeof(float), sort_sm = ((size_t)3 * E + 1) * sizeof(int);
    if (route_sm > 96 * 1024 || sort_sm > 48 * 1024) return KP_ERR_UNSUPPORTED;            // (E <= 1536)
    cudaStream_t s = (cudaStream_t)stream;
    if (route_sm > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)route_sm);
        if (e != cudaSuccess) return (int)e;
    }
    kp_launch_pdl(moe_route_kernel, dim3((n + 7) / 8), dim3(256), route_sm, s, logits, bias, n, E, top, mode, wscale, idx, weights);
    cudaError_t e0 = cudaGetLastError();
    if (e0 != cudaSuccess) return (int)e0;
    int* offsets = layout;
    int* tile_start = offsets + (E + 1);
    int* big_start = tile_start + (E + 1);
    int* perm = big_start + (E + 1);
    int* inv = perm + (size_t)n * top;
    kp_launch_pdl(moe_sort_kernel, dim3(1), dim3(MOE_SORT_THREADS), sort_sm, s, (const int*)idx, n * top, E, E - n_identity, offsets,
                  tile_start, big_start, perm, inv);
    return kp_launch_status();
}

// The router in one go: rows h [n, d] (storage type `dtype`), Wr [E, d] and b [E] (or null) in float32 -> idx, weights
// and the layout.  KP_ERR_UNSUPPORTED where the rows do not fit the kernel's shared memory or alignment (the caller
// then computes the logits with a matrix product and calls kp_moe_route).
int kp_moe_router(const void* h, int ldh, const float* wr, const float* bias, int n, int E, int d, int top, int mode,
                  float wscale, int n_identity, int* idx, float* weights, int* layout, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (E < 1 || top < 1 || top > E || top > MOE_MAX_TOP || mode < 0 || mode > 2 || n_identity < 0 || n_identity >= E)
        return KP_ERR_UNSUPPORTED;
    const size_t sort_sm = ((size_t)3 * E + 1) * sizeof(int);
    // eight rows a block where there are many and they fit shared memory, else one
    const int rb = (n > 64 && ((size_t)8 * (d + 2 * E)) * sizeof(float) <= 200 * 1024) ? 8 : 1;
    const size_t sm = ((size_t)rb * d + (size_t)rb * 2 * E) * sizeof(float);
    if ((d & 3) || ((uintptr_t)wr & 15) || sm > 200 * 1024 || sort_sm > 48 * 1024) return KP_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
#define MOE_ROUTER_LAUNCH(T, RB)                                                                                          \
    do {                                                                                                                  \
        if (sm > 48 * 1024) {                                                                                             \
            cudaError_t e = cudaFuncSetAttribute(moe_router_kernel<T, RB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm); \
            if (e != cudaSuccess) return (int)e;                                                                          \
        }                                                                                                                 \
        kp_launch_pdl(moe_router_kernel<T, RB>, dim3((n + RB - 1) / RB), dim3(256), sm, s, (const T*)h, ldh, wr, bias, n, E, d, \
                      top, mode, wscale, idx, weights);                                                                   \
    } while (0)
    KP_DISPATCH_DTYPE(dtype, T, { if (rb == 8) MOE_ROUTER_LAUNCH(T, 8); else MOE_ROUTER_LAUNCH(T, 1); });
#undef MOE_ROUTER_LAUNCH
    cudaError_t e0 = cudaGetLastError();
    if (e0 != cudaSuccess) return (int)e0;
    int* offsets = layout;
    int* tile_start = offsets + (E + 1);
    int* big_start = tile_start + (E + 1);
    int* perm = big_start + (E + 1);
    int* inv = perm + (size_t)n * top;
    kp_launch_pdl(moe_sort_kernel, dim3(1), dim3(MOE_SORT_THREADS), sort_sm, s, (const int*)idx, n * top, E, E - n_identity, offsets,
                  tile_start, big_start, perm, inv);
    return kp_launch_status();
}

// h [n, d] -> act [n top, ff] (by place) -> y [n top, d] float32 (by place) -> out [n, d] += weighted sum.
// hs: scratch [n top, d] in the storage type for the tcgen05 path (null: that path is not taken).
// E counts all router outputs; the last n_identity of them are experts without weights (w_gu and w_down hold
// E - n_identity experts), for which `idx` [n, top] (the chosen experts) must be given.
// weight_input: the weights multiply the experts' inputs (hs is then needed whatever the path; no identity experts).
int kp_moe_experts_weighted(const void* h, int ldh, const void* w_gu, const void* w_down, const int* layout, const float* weights,
                            void* act, float* y, float* out, void* hs, int n, int E, int top, int d, int ff, int act_kind, int dtype,
                            int n_identity, const int* idx, int weight_input, void* stream) {
    if (n <= 0) return 0;
    if (weight_input && (hs == nullptr || n_identity > 0)) return KP_ERR_BAD_ARG;
    if (E < 1 || top < 1 || d < 1 || ff < 1 || act_kind < 0 || act_kind > KP_ACT_GELU_TANH) return KP_ERR_BAD_ARG;
    if (n_identity < 0 || n_identity >= E || (n_identity > 0 && idx == nullptr)) return KP_ERR_BAD_ARG;
    const int E_real = E - n_identity;
    const int max_tiles = kp_moe_max_tiles(n, E, top);
    if (max_tiles > 65535) return KP_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int* offsets = layout;
    const int* tile_start = offsets + (E + 1);
    const int* big_start = tile_start + (E + 1);
    const int* perm = big_start + (E + 1);
    const int* inv = perm + (size_t)n * top;
    cudaError_t e0;
    const bool tc = dtype == KP_DTYPE_BF16 && d % 8 == 0 && ff % 8 == 0 && ldh % 8 == 0 &&
                    !(((uintptr_t)h | (uintptr_t)w_gu | (uintptr_t)w_down | (uintptr_t)act) & 15) &&
                    !(weight_input && ((uintptr_t)hs & 15));
    const long long pairs = (long long)n * top;
    const void* rows = h;                          // what the grouped products of the smaller tiles read, and how
    int ld_rows = ldh;
    const int* perm_rows = perm;
    bool gathered = false;
    if (weight_input) {
        size_t gg = ((size_t)pairs * (tc ? d / 8 : d) + 255) / 256;
        if (gg > 148 * 16) gg = 148 * 16;
        if (tc) {
            kp_launch_pdl(moe_gather_scaled_vec_kernel, dim3((unsigned)gg), dim3(256), 0, s, (const bf16*)h, ldh, perm, weights,
                          (bf16*)hs, (int)pairs, d / 8, top);
        } else {
            KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(moe_gather_scaled_kernel<T>, dim3((unsigned)gg), dim3(256), 0, s, (const T*)h,
                                                       ldh, perm, weights, (T*)hs, (int)pairs, d, top)));
        }
        if ((e0 = cudaGetLastError()) != cudaSuccess) return (int)e0;
        rows = hs; ld_rows = d; perm_rows = nullptr; gathered = true;
        weights = nullptr;
    }
    const long long big_tiles = pairs / MOE_BIG + (pairs < E ? pairs : E);
    if (tc && hs != nullptr && pairs >= g_moe_tc_min_pairs && big_tiles <= 65535 && !((uintptr_t)hs & 15) &&
        (long long)E_real * 2 * ff < 2147483647LL && (long long)E_real * d < 2147483647LL) {
        // many rows an expert: the tcgen05 tiles
        alignas(64) CUtensorMap ta1, tw1, ta2, tw2;
        int st = kp_make_map_bf16_2d(&ta1, hs, (unsigned long long)pairs, d, d, MT_BK, MOE_BIG);
        if (!st) st = kp_make_map_bf16_2d(&tw1, w_gu, (unsigned long long)E_real * 2 * ff, d, d, MT_BK, MT_BN / 2);
        if (!st) st = kp_make_map_bf16_2d(&ta2, act, (unsigned long long)pairs, ff, ff, MT_BK, MOE_BIG);
        if (!st) st = kp_make_map_bf16_2d(&tw2, w_down, (unsigned long long)E_real * d, ff, ff, MT_BK, MT_BN);
        if (st) return st;
        const size_t smem = (size_t)MT_STAGES * (MT_A_BYTES + MT_B_BYTES) + (2 * MT_STAGES + 1) * 8 + 16 + 1024;
        static bool ready = false;
        if (!ready) {
            if ((e0 = cudaFuncSetAttribute(moe_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return (int)e0;
            if ((e0 = cudaFuncSetAttribute(moe_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return (int)e0;
            ready = true;
        }
        size_t gg = ((size_t)pairs * (d / 8) + 255) / 256;
        if (gg > 148 * 16) gg = 148 * 16;
        if (!gathered) {
            kp_launch_pdl(moe_gather_rows_kernel, dim3((unsigned)gg), dim3(256), 0, s, (const bf16*)h, ldh, perm, (bf16*)hs, (int)pairs,
                          d / 8, top);
            if ((e0 = cudaGetLastError()) != cudaSuccess) return (int)e0;
        }
        MtArgs a1 = {offsets, big_start, E, d, ff, 2 * ff, ff, act, ff, act_kind};
        kp_launch_pdl(moe_tc_kernel<true>, dim3((ff + MT_BN / 2 - 1) / (MT_BN / 2), (unsigned)big_tiles), dim3(MT_THREADS), smem, s,
                      ta1, tw1, a1);
        if ((e0 = cudaGetLastError()) != cudaSuccess) return (int)e0;
        MtArgs a2 = {offsets, big_start, E, ff, d, d, 0, y, d, 0};
        kp_launch_pdl(moe_tc_kernel<false>, dim3((d + MT_BN - 1) / MT_BN, (unsigned)big_tiles), dim3(MT_THREADS), smem, s, ta2, tw2, a2);
        if ((e0 = cudaGetLastError()) != cudaSuccess) return (int)e0;
    } else if (tc) {
        kp_launch_pdl(moe_gate_up_tc_kernel, dim3((ff + MOE_TC_BN - 1) / MOE_TC_BN, max_tiles), dim3(128), 0, s, (const bf16*)rows,
                      ld_rows, (const bf16*)w_gu, offsets, tile_start, perm_rows, (bf16*)act, E, top, d, ff, act_kind);
        if ((e0 = cudaGetLastError()) != cudaSuccess) return (int)e0;
        kp_launch_pdl(moe_down_tc_kernel, dim3((d + MOE_TC_BN - 1) / MOE_TC_BN, max_tiles), dim3(128), 0, s, (const bf16*)act,
                      (const bf16*)w_down, offsets, tile_start, y, E, d, ff);
        if ((e0 = cudaGetLastError()) != cudaSuccess) return (int)e0;
    } else {
        KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(moe_gate_up_kernel<T>, dim3((ff + 31) / 32, max_tiles), dim3(256), 0, s,
                                                   (const T*)rows, ld_rows, (const T*)w_gu, offsets, tile_start, perm_rows, (T*)act, E, top,
                                                   d, ff, act_kind)));
        if ((e0 = cudaGetLastError()) != cudaSuccess) return (int)e0;
        KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(moe_down_kernel<T>, dim3((d + 63) / 64, max_tiles), dim3(256), 0, s,
                                                   (const T*)act, (const T*)w_down, offsets, tile_start, y, E, d, ff)));
        if ((e0 = cudaGetLastError()) != cudaSuccess) return (int)e0;
    }
    size_t g = ((size_t)n * d + 255) / 256;
    if (g > 148 * 16) g = 148 * 16;
    if (n_identity > 0) {
        KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(moe_combine_identity_kernel<T>, dim3((unsigned)g), dim3(256), 0, s, (const float*)y,
                                                   inv, weights, idx, (const T*)h, ldh, E_real, out, n, d, top)));
        return kp_launch_status();
    }
    kp_launch_pdl(moe_combine_kernel, dim3((unsigned)g), dim3(256), 0, s, (const float*)y, inv, weights, out, n, d, top);
    return kp_launch_status();
}

int kp_moe_experts(const void* h, int ldh, const void* w_gu, const void* w_down, const int* layout, const float* weights,
                   void* act, float* y, float* out, void* hs, int n, int E, int top, int d, int ff, int act_kind, int dtype,
                   int n_identity, const int* idx, void* stream) {
    return kp_moe_experts_weighted(h, ldh, w_gu, w_down, layout, weights, act, y, out, hs, n, E, top, d, ff, act_kind, dtype,
                                   n_identity, idx, 0, stream);
}

}  // extern "C"
