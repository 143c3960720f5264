// Split-KV attention for rows that each read a long cache (decode steps and
// very short portions): the keys of one (row, kv head) are cut into chunks of
// 256 at multiples of 256 of the absolute key index; one CTA per (chunk, kv
// head, row) computes, for all R = H/G query heads that share the kv head, the
// chunk's scores, its maximum m, its sum l of exp(s - m) and the unnormalised
// sum of exp(s - m) V; a second kernel merges the chunks of a row in order.
// Same formulas as attention.cu (src/backend/cpu/scalar/core.c:383-433); the
// chunk grid does not depend on the batch, so neither does the result.
//
// Scratch (global memory beyond inputs and outputs, given by the caller):
//   part_acc [n_rows][H][n_chunks][hd] float, part_ml [n_rows][H][n_chunks][2] float.
// Only the chunks that intersect a row's key range are written and read.
//
// Two variants, each an argument.  `keep_first` > 0: behind a window a row also reads the keys 0 .. keep_first - 1
// of its sequence; the chunks that hold them are computed and merged in front of the window's chunks, the chunks
// in between are skipped.  Where another kernel computes the window's chunks (the tensor-core form, which knows
// nothing of kept keys), a second small launch of the kernel below (`front`) computes the kept keys alone, into slots
// of their own behind the window's chunks (`slot0` on), and the merge is told where they are.  `sink` (one float32 number a query head, or null): exp(sink_h) is added to the softmax's
// denominator, once a row, by the merge (the chunk kernels know nothing of it).
#include "common.cuh"

#define AD_CHUNK 256
#define AD_THREADS 256
#define AD_RMAX 8
#define KP_MAX_HEAD_DIM 256

template <typename T> struct Vec16;
template <> struct Vec16<bf16> { static constexpr int N = 8; };
template <> struct Vec16<float> { static constexpr int N = 4; };

template <typename T>
__device__ __forceinline__ void unpack16(const uint4& v, float* f);
template <>
__device__ __forceinline__ void unpack16<bf16>(const uint4& v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
template <>
__device__ __forceinline__ void unpack16<float>(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
}

// The keys a row at position `pos` reads: the last `window` ones (window > 0), and with block > 0 none from
// before the start of its own block of `block` positions, blocks being counted from position 0 of the sequence.
__device__ __forceinline__ void key_range(int pos, int window, int block, int& k_lo, int& k_hi) {
    k_lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (block > 0) k_lo = max(k_lo, (pos / block) * block);
    k_hi = pos;
}
// The chunks a row's merge walks: those that hold kept first keys (keys below first_hi = min(keep_first, k_lo)) and
// lie before the window's first chunk c_lo, then c_lo .. c_hi.  n_front of the first kind; the i-th of all is
// chunk_at(i, ...).
__device__ __forceinline__ int front_chunks(int first_hi, int chunk_keys, int c_lo) {
    return min(c_lo, (first_hi + chunk_keys - 1) / chunk_keys);
}
__device__ __forceinline__ int chunk_at(int i, int n_front, int c_lo, int front_slot0 = -1) {
    return i < n_front ? (front_slot0 >= 0 ? front_slot0 + i : i) : c_lo + (i - n_front);
}
// (front_slot0 >= 0: the kept keys' chunks, of AD_CHUNK keys each, lie in slots of their own and hold kept keys only)
#define AD_CHUNK_KEYS 256
__device__ __forceinline__ int merge_front(int first_hi, int chunk_keys, int c_lo, int front_slot0) {
    return front_slot0 >= 0 ? (first_hi + AD_CHUNK_KEYS - 1) / AD_CHUNK_KEYS : front_chunks(first_hi, chunk_keys, c_lo);
}

// HD, RR: head size and query heads per kv head fixed at compile time (loops unroll, loads overlap);
// 0 means "taken from the arguments".
template <typename T, int HD, int RR>
__global__ void __launch_bounds__(AD_THREADS)
attn_split_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ cache, const int* __restrict__ block_table,
                  int max_blocks, const int* __restrict__ row_seg, const int* __restrict__ positions,
                  float* __restrict__ part_acc, float* __restrict__ part_ml, int n_chunks, float scale, int window,
                  int page_size, int H, int G, int hd_rt, int block, int keep_first, int slot0, int front) {
    kp_pdl_begin();
    extern __shared__ float smem[];
    const int hd = HD ? HD : hd_rt;
    const int R = RR ? RR : H / G;
    float* qs = smem;                              // [R][hd]
    float* ps = qs + R * hd;                       // [R][AD_CHUNK]
    float* red = ps + R * AD_CHUNK;                // [n_slices][R][hd]  (also used for the small reductions)
    __shared__ float wred[AD_THREADS / 32][AD_RMAX];
    __shared__ float stat_m[AD_RMAX], stat_l[AD_RMAX];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int chunk = blockIdx.x, g = blockIdx.y, row = blockIdx.z;
    int k_lo, k_hi;
    key_range(positions[row], window, block, k_lo, k_hi);
    const int c0 = chunk * AD_CHUNK;
    int first_hi = min(keep_first, k_lo);                       // keys below it are read although they lie before the window
    if (front) { k_hi = first_hi - 1; k_lo = 0; first_hi = 0; } // the kept keys alone (none: no chunk passes the test below)
    if (c0 > k_hi || (c0 + AD_CHUNK - 1 < k_lo && c0 >= first_hi)) return;          // the chunk holds none of this row's keys
    const int* bt = block_table + (size_t)row_seg[row] * max_blocks;
    const size_t page_stride = (size_t)2 * G * page_size * hd;
    const size_t k_off = (size_t)g * page_size * hd, v_off = ((size_t)G + g) * page_size * hd;

    for (int i = tid; i < R * hd; i += AD_THREADS)
        qs[i] = to_f32(q[(size_t)row * ldq + (size_t)(g * R) * hd + i]);
    __syncthreads();

    // (head size 64, 16-bit cache) the values this thread multiplies later are fetched now, so that their
    // latency passes under the scores and the softmax: thread = (pair of dims, slice of 32 keys)
    constexpr bool PREFETCH_V = (HD == 64) && (sizeof(T) == 2);
    uint32_t vpre[PREFETCH_V ? 32 : 1];
    if (PREFETCH_V) {
        const int pair_p = tid & 31, slice_p = tid >> 5;
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const int key2 = c0 + slice_p * 32 + j;
            uint32_t v = 0;
            if (key2 <= k_hi && (key2 >= k_lo || key2 < first_hi))
                v = *reinterpret_cast<const uint32_t*>(cache + (size_t)bt[key2 / page_size] * page_stride + v_off +
                                                       (size_t)(key2 % page_size) * hd + 2 * pair_p);
            vpre[j] = v;
        }
    }

    // scores: one key a thread, all R heads
    const int key = c0 + tid;
    const bool valid = key <= k_hi && (key >= k_lo || key < first_hi);
    float s[AD_RMAX];
#pragma unroll
    for (int r = 0; r < AD_RMAX; r++) s[r] = 0.f;
    if (valid) {
        const T* kp = cache + (size_t)bt[key / page_size] * page_stride + k_off + (size_t)(key % page_size) * hd;
        constexpr int VN = Vec16<T>::N;
#pragma unroll
        for (int i = 0; i < hd; i += VN) {
            float kf[VN];
            unpack16<T>(*reinterpret_cast<const uint4*>(kp + i), kf);
#pragma unroll
            for (int r = 0; r < AD_RMAX; r++) {
                if (r < R) {
                    const float* qr = qs + r * hd + i;
#pragma unroll
                    for (int j = 0; j < VN; j++) s[r] = fmaf(qr[j], kf[j], s[r]);
                }
            }
        }
    }
    // per head: chunk maximum, exp, chunk sum
#pragma unroll
    for (int r = 0; r < AD_RMAX; r++) {
        if (r < R) {
            s[r] = valid ? s[r] * scale : -INFINITY;
            const float m = warp_max(s[r]);
            if (lane == 0) wred[warp][r] = m;
        }
    }
    __syncthreads();
    if (tid < R) {
        float m = wred[0][tid];
        for (int w = 1; w < AD_THREADS / 32; w++) m = fmaxf(m, wred[w][tid]);
        stat_m[tid] = m;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < AD_RMAX; r++) {
        if (r < R) {
            const float p = valid ? expf(s[r] - stat_m[r]) : 0.f;
            ps[r * AD_CHUNK + tid] = p;
            const float l = warp_sum(p);
            if (lane == 0) wred[warp][r] = l;
        }
    }
    __syncthreads();
    if (tid < R) {
        float l = 0.f;
        for (int w = 0; w < AD_THREADS / 32; w++) l += wred[w][tid];
        stat_l[tid] = l;
    }

    // P V: thread = (pair of dims, slice of keys); slices are summed in order afterwards
    const int pairs = hd >> 1;
    const int n_slices = AD_THREADS / pairs;
    const int per = (AD_CHUNK + n_slices - 1) / n_slices;
    const int pair = tid % pairs, slice = tid / pairs;
    float acc[AD_RMAX][2];
#pragma unroll
    for (int r = 0; r < AD_RMAX; r++) acc[r][0] = acc[r][1] = 0.f;
    if (PREFETCH_V) {
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const int kk = slice * 32 + j;                       // keys outside the row's range have p = 0
            const float v0 = __uint_as_float(vpre[j] << 16), v1 = __uint_as_float(vpre[j] & 0xffff0000u);
#pragma unroll
            for (int r = 0; r < AD_RMAX; r++) {
                if (r < R) {
                    const float p = ps[r * AD_CHUNK + kk];
                    acc[r][0] = fmaf(p, v0, acc[r][0]);
                    acc[r][1] = fmaf(p, v1, acc[r][1]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < AD_RMAX; r++) {
            if (r < R) {
                red[((size_t)slice * R + r) * hd + 2 * pair] = acc[r][0];
                red[((size_t)slice * R + r) * hd + 2 * pair + 1] = acc[r][1];
            }
        }
    } else if (slice < n_slices) {
        const int kk_lo = max(slice * per, first_hi > c0 ? 0 : k_lo - c0), kk_hi = min(min((slice + 1) * per, AD_CHUNK) - 1, k_hi - c0);
#pragma unroll 8
        for (int kk = kk_lo; kk <= kk_hi; kk++) {
            const int key2 = c0 + kk;
            if (key2 < k_lo && key2 >= first_hi) continue;
            const T* vp = cache + (size_t)bt[key2 / page_size] * page_stride + v_off +
                          (size_t)(key2 % page_size) * hd + 2 * pair;
            const float v0 = to_f32(vp[0]), v1 = to_f32(vp[1]);
#pragma unroll
            for (int r = 0; r < AD_RMAX; r++) {
                if (r < R) {
                    const float p = ps[r * AD_CHUNK + kk];
                    acc[r][0] = fmaf(p, v0, acc[r][0]);
                    acc[r][1] = fmaf(p, v1, acc[r][1]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < AD_RMAX; r++) {
            if (r < R) {
                red[((size_t)slice * R + r) * hd + 2 * pair] = acc[r][0];
                red[((size_t)slice * R + r) * hd + 2 * pair + 1] = acc[r][1];
            }
        }
    }
    __syncthreads();
    for (int e = tid; e < R * hd; e += AD_THREADS) {
        const int r = e / hd, d = e % hd;
        float v = 0.f;
        for (int sl = 0; sl < n_slices; sl++) v += red[((size_t)sl * R + r) * hd + d];
        part_acc[(((size_t)row * H + g * R + r) * n_chunks + slot0 + chunk) * hd + d] = v;
    }
    if (tid < R) {
        float* ml = part_ml + (((size_t)row * H + g * R + tid) * n_chunks + slot0 + chunk) * 2;
        ml[0] = stat_m[tid];
        ml[1] = stat_l[tid];
    }
}

#define MERGE_THREADS 256
#define MERGE_BATCH 4096                                    // floats of accumulators in shared memory at a time

// The chunks of a row and head put together: out = sum_c acc_c * exp(m_c - m) / sum_c l_c * exp(m_c - m), the
// sums in chunk order.  One CTA a (head, row).  The statistics of the row's chunks and the weights
// exp(m_c - m) are brought into shared memory once by all threads together; only the sums themselves run
// chunk by chunk (a context of 32k tokens has 128 chunks: with every thread walking global memory three times
// for them the merge took longer than half of the attention itself).
template <typename T>
__global__ void attn_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                  const int* __restrict__ positions, T* __restrict__ out, int ldo, int n_chunks,
                                  int chunk_keys, int window, int H, int hd, int block, int keep_first,
                                  const float* __restrict__ sink, int front_slot0) {
    kp_pdl_begin_early_if(gridDim.y > 1);
    extern __shared__ __align__(16) float merge_sm[];       // [MERGE_BATCH], [n_chunks] l_c, [n_chunks] exp(m_c - m), [32]
    const int h = blockIdx.x, row = blockIdx.y, tid = threadIdx.x, nt = blockDim.x;
    int k_lo, k_hi;
    key_range(positions[row], window, block, k_lo, k_hi);
    // (a position beyond the chunks the caller gave is the caller's fault; the clamp keeps the reads inside
    // the scratch and the shared arrays all the same)
    const int c_hi = min(k_hi / chunk_keys, n_chunks - 1), c_lo = min(k_lo / chunk_keys, c_hi);
    const int n_front = merge_front(min(keep_first, k_lo), chunk_keys, c_lo, front_slot0), n = n_front + c_hi - c_lo + 1;
    float* s_acc = merge_sm;
    float* s_l = merge_sm + MERGE_BATCH;
    float* s_w = s_l + n_chunks;
    float* s_red = s_w + n_chunks;
    // the accumulators: brought in batches of MERGE_BATCH floats by all threads (every load of a batch in
    // flight at once), then added chunk by chunk by the thread of each dimension
    const float* pa = part_acc + ((size_t)row * H + h) * n_chunks * hd;
    const int mb = MERGE_BATCH / hd;                        // chunks a batch
    constexpr int PER = MERGE_BATCH / 4 / MERGE_THREADS;    // float4 a thread and batch
    float4 reg[PER];
    auto fetch = [&](int c0) {                              // the batch from chunk c0 on, into registers
        const int nb = min(mb, n - c0);
#pragma unroll
        for (int k = 0; k < PER; k++) {
            const int i = (k * MERGE_THREADS + tid) * 4;
            if (i < nb * hd) {
                const int j = i / hd;                       // (hd is a multiple of 4: a float4 stays inside one chunk)
                reg[k] = *reinterpret_cast<const float4*>(pa + (size_t)chunk_at(c0 + j, n_front, c_lo, front_slot0) * hd + (i - j * hd));
            }
        }
    };
    fetch(0);                                               // under way while the statistics are worked out
    const float* ml = part_ml + ((size_t)row * H + h) * n_chunks * 2;
    float m = -INFINITY;
    for (int c = tid; c < n; c += nt) {
        const float2 v = *reinterpret_cast<const float2*>(ml + 2 * chunk_at(c, n_front, c_lo, front_slot0));
        s_w[c] = v.x;                                       // m_c for now
        s_l[c] = v.y;
        m = fmaxf(m, v.x);
    }
    m = warp_max(m);
    if ((tid & 31) == 0) s_red[tid >> 5] = m;
    __syncthreads();
    m = -INFINITY;
    for (int w = 0; w < (nt + 31) / 32; w++) m = fmaxf(m, s_red[w]);
    if (sink) m = fmaxf(m, sink[h]);
    for (int c = tid; c < n; c += nt) s_w[c] = expf(s_w[c] - m);
    __syncthreads();
    float l = sink ? expf(sink[h] - m) : 0.f;               // the sink: in the denominator once, with no value
    for (int c = 0; c < n; c++) l = __fmaf_rn(s_l[c], s_w[c], l);
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    float v = 0.f;
    for (int c0 = 0; c0 < n; c0 += mb) {
        const int nb = min(mb, n - c0);
#pragma unroll
        for (int k = 0; k < PER; k++) {
            const int i = (k * MERGE_THREADS + tid) * 4;
            if (i < nb * hd) *reinterpret_cast<float4*>(s_acc + i) = reg[k];
        }
        __syncthreads();
        if (c0 + mb < n) fetch(c0 + mb);                    // the next batch is under way while this one is added
        if (tid < hd)
            for (int j = 0; j < nb; j++) v = fmaf(s_acc[j * hd + tid], s_w[c0 + j], v);
        __syncthreads();
    }
    if (tid < hd) out[(size_t)row * ldo + (size_t)h * hd + tid] = from_f32<T>(v * inv);
}

// The same for rows of at most 64 chunks (16k keys), one warp a (head, row) and no shared memory: the lanes
// hold the chunks' statistics and weights and pass them round, every lane sums its dimensions (lane, lane + 32,
// ...) chunk by chunk.  The arithmetic is that of the kernel above, so a row's result does not depend on which
// of the two ran.  (With 64 rows the kernel above took 10.7 us for 2048 small CTAs of 256 threads.)
#define MERGE_WARP_CHUNKS 64
#define MERGE_WARP_BLOCK 16                               // chunks whose sums a warp fetches at a time
template <typename T>
__global__ void attn_merge_warp_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                       const int* __restrict__ positions, T* __restrict__ out, int ldo, int n_chunks,
                                       int chunk_keys, int window, int H, int hd, int n_rows, int block, int keep_first,
                                       const float* __restrict__ sink, int front_slot0) {
    kp_pdl_begin_early_if(n_rows > 1);
    const int lane = threadIdx.x & 31;
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);          // (row, head)
    if (item >= n_rows * H) return;
    const int row = item / H, h = item - row * H;
    int k_lo, k_hi;
    key_range(positions[row], window, block, k_lo, k_hi);
    const int c_hi = min(k_hi / chunk_keys, n_chunks - 1), c_lo = min(k_lo / chunk_keys, c_hi);
    const int n_front = merge_front(min(keep_first, k_lo), chunk_keys, c_lo, front_slot0), n = n_front + c_hi - c_lo + 1;
    const float* pa = part_acc + ((size_t)row * H + h) * n_chunks * hd;
    const float* ml = part_ml + ((size_t)row * H + h) * n_chunks * 2;
    // the sums of the first MERGE_WARP_BLOCK chunks are on their way while the statistics are worked out
    constexpr int B = MERGE_WARP_BLOCK;
    float a[B][4];
    auto fetch = [&](int c0) {
#pragma unroll
        for (int j = 0; j < B; j++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int d = lane + 32 * i;
                a[j][i] = (c0 + j < n && d < hd) ? pa[(size_t)chunk_at(c0 + j, n_front, c_lo, front_slot0) * hd + d] : 0.f;
            }
    };
    fetch(0);
    float m0 = -INFINITY, l0 = 0.f, m1 = -INFINITY, l1 = 0.f;                       // chunks lane and lane + 32
    if (lane < n) { const float2 v = *reinterpret_cast<const float2*>(ml + 2 * chunk_at(lane, n_front, c_lo, front_slot0)); m0 = v.x; l0 = v.y; }
    if (lane + 32 < n) { const float2 v = *reinterpret_cast<const float2*>(ml + 2 * chunk_at(lane + 32, n_front, c_lo, front_slot0)); m1 = v.x; l1 = v.y; }
    float m = warp_max(fmaxf(m0, m1));
    if (sink) m = fmaxf(m, sink[h]);
    const float w0 = lane < n ? expf(m0 - m) : 0.f, w1 = lane + 32 < n ? expf(m1 - m) : 0.f;
    float l = sink ? expf(sink[h] - m) : 0.f, v[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c0 = 0; c0 < n; c0 += B) {
        if (c0) fetch(c0);
#pragma unroll
        for (int j = 0; j < B; j++) {
            const int c = c0 + j;
            if (c < n) {                                                            // (the same for all lanes)
                const float wc = __shfl_sync(0xffffffffu, c < 32 ? w0 : w1, c & 31);
                const float lc = __shfl_sync(0xffffffffu, c < 32 ? l0 : l1, c & 31);
                l = __fmaf_rn(lc, wc, l);
#pragma unroll
                for (int i = 0; i < 4; i++) v[i] = fmaf(a[j][i], wc, v[i]);
            }
        }
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int d = lane + 32 * i;
        if (d < hd) out[(size_t)row * ldo + (size_t)h * hd + d] = from_f32<T>(v[i] * inv);
    }
}

static size_t merge_smem_bytes(int n_chunks) { return sizeof(float) * ((size_t)2 * n_chunks + 32 + MERGE_BATCH); }

template <typename T>
static int launch_merge(const float* part_acc, const float* part_ml, const int* positions, void* out, int ldo,
                        int n_chunks, int chunk_keys, int window, int block, int keep_first, const float* sink, int n, int H,
                        int hd, cudaStream_t s, int front_slot0 = -1) {
    if (window <= 0) keep_first = 0;
    if (keep_first == 0) front_slot0 = -1;
    if (n_chunks <= MERGE_WARP_CHUNKS && hd <= 128) {
        const int warps = 8;
        kp_launch_pdl(attn_merge_warp_kernel<T>, dim3((n * H + warps - 1) / warps), dim3(warps * 32), 0, s, part_acc, part_ml,
                      positions, (T*)out, ldo, n_chunks, chunk_keys, window, H, hd, n, block, keep_first, sink, front_slot0);
        return kp_launch_status();
    }
    const size_t smem = merge_smem_bytes(n_chunks);
    if (smem > 200 * 1024) return KP_ERR_UNSUPPORTED;       // (25,000 chunks: 6.5 million keys)
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attn_merge_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    if (hd > MERGE_THREADS || (hd & 3)) return KP_ERR_UNSUPPORTED;
    kp_launch_pdl(attn_merge_kernel<T>, dim3(H, n), dim3(MERGE_THREADS), smem, s, part_acc, part_ml, positions, (T*)out, ldo,
                  n_chunks, chunk_keys, window, H, hd, block, keep_first, sink, front_slot0);
    return kp_launch_status();
}

static size_t split_smem_bytes(int R, int hd) {
    const int pairs = hd / 2;
    const int n_slices = AD_THREADS / pairs;
    return sizeof(float) * ((size_t)R * hd + (size_t)R * AD_CHUNK + (size_t)n_slices * R * hd);
}

extern "C" {

// Elements of float scratch the split kernel needs for these sizes (part_acc then part_ml).
long long kp_attention_split_scratch(int n_rows, int H, int hd, int n_chunks) {
    return (long long)n_rows * H * n_chunks * (hd + 2);
}

// n_chunks: chunks of 256 keys the grid covers; must reach the largest position in the batch.
// block: 0, or the size of the blocks of positions that a row's keys do not reach beyond (see key_range).
// keep_first: the first keys of the sequence that stay readable behind a window; sink: [H] float32 or null.
int kp_attention_split_sink(const void* q, int ldq, const void* cache, const int* block_table, int max_blocks,
                            const int* row_seg, const int* positions, void* out, int ldo, float* scratch, int n_chunks,
                            float scale, int window, int block, int keep_first, const float* sink, int page_size, int n,
                            int H, int G, int hd, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (keep_first < 0 || (keep_first > 0 && block > 0)) return KP_ERR_BAD_ARG;
    if (window <= 0) keep_first = 0;
    if (hd < 16 || hd > KP_MAX_HEAD_DIM || (hd & 15)) return KP_ERR_UNSUPPORTED;
    if (G < 1 || H % G != 0 || H / G > AD_RMAX || page_size < 1 || n_chunks < 1) return KP_ERR_UNSUPPORTED;
    if (n > 65535 || G > 65535) return KP_ERR_UNSUPPORTED;
    const int R = H / G;
    const size_t smem = split_smem_bytes(R, hd);
    float* part_acc = scratch;
    float* part_ml = scratch + (size_t)n * H * n_chunks * hd;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_chunks, G, n);
    constexpr int SLOT0 = 0, FRONT = 0;
#define AD_LAUNCH(T, HD, RR)                                                                                      \
    kp_launch_pdl(attn_split_kernel<T, HD, RR>, dim3(grid), dim3(AD_THREADS), smem, s, (const T*)q, ldq, (const T*)cache, block_table,       \
                                                                max_blocks, row_seg, positions, part_acc, part_ml,    \
                                                                n_chunks, scale, window, page_size, H, G, hd, block, keep_first, SLOT0, FRONT)
    KP_DISPATCH_DTYPE(dtype, T, {
        cudaError_t e0;
        if (hd == 64 && R == 4) e0 = AD_LAUNCH(T, 64, 4);
        else if (hd == 64) e0 = AD_LAUNCH(T, 64, 0);
        else if (hd == 128) e0 = AD_LAUNCH(T, 128, 0);
        else e0 = AD_LAUNCH(T, 0, 0);
        if (e0 != cudaSuccess) { cudaGetLastError(); return (int)e0; }      // the first launch that failed
        return launch_merge<T>(part_acc, part_ml, positions, out, ldo, n_chunks, AD_CHUNK, window, block, keep_first, sink, n, H, hd, s);
    });
#undef AD_LAUNCH
    return kp_launch_status();
}

int kp_attention_split_masked(const void* q, int ldq, const void* cache, const int* block_table, int max_blocks,
                              const int* row_seg, const int* positions, void* out, int ldo, float* scratch, int n_chunks,
                              float scale, int window, int block, int page_size, int n, int H, int G, int hd, int dtype,
                              void* stream) {
    return kp_attention_split_sink(q, ldq, cache, block_table, max_blocks, row_seg, positions, out, ldo, scratch, n_chunks,
                                   scale, window, block, 0, nullptr, page_size, n, H, G, hd, dtype, stream);
}

int kp_attention_split(const void* q, int ldq, const void* cache, const int* block_table, int max_blocks,
                       const int* row_seg, const int* positions, void* out, int ldo, float* scratch, int n_chunks,
                       float scale, int window, int page_size, int n, int H, int G, int hd, int dtype, void* stream) {
    return kp_attention_split_masked(q, ldq, cache, block_table, max_blocks, row_seg, positions, out, ldo, scratch,
                                     n_chunks, scale, window, 0, page_size, n, H, G, hd, dtype, stream);
}

// The merge alone, for partials of chunks of `chunk_keys` keys that another kernel wrote into `scratch` in the
// same format.
// The kept first keys alone, for partials whose window chunks another kernel writes: chunks of 256 keys into the slots
// front_slot0, front_slot0 + 1, ... of a scratch of n_chunks slots a (row, head).  The merge is then given front_slot0.
int kp_attention_front_chunks(const void* q, int ldq, const void* cache, const int* block_table, int max_blocks,
                              const int* row_seg, const int* positions, float* scratch, int n_chunks, int front_slot0, float scale,
                              int window, int keep_first, int page_size, int n, int H, int G, int hd, int dtype, void* stream) {
    if (n <= 0 || keep_first <= 0 || window <= 0) return 0;
    if (hd < 16 || hd > KP_MAX_HEAD_DIM || (hd & 15)) return KP_ERR_UNSUPPORTED;
    if (G < 1 || H % G != 0 || H / G > AD_RMAX || page_size < 1 || n > 65535 || G > 65535) return KP_ERR_UNSUPPORTED;
    const int n_front = (keep_first + AD_CHUNK - 1) / AD_CHUNK;
    if (front_slot0 < 0 || front_slot0 + n_front > n_chunks) return KP_ERR_BAD_ARG;
    const size_t smem = split_smem_bytes(H / G, hd);
    float* part_acc = scratch;
    float* part_ml = scratch + (size_t)n * H * n_chunks * hd;
    KP_DISPATCH_DTYPE(dtype, T, (kp_launch_pdl(attn_split_kernel<T, 0, 0>, dim3(n_front, G, n), dim3(AD_THREADS), smem, (cudaStream_t)stream,
                                               (const T*)q, ldq, (const T*)cache, block_table, max_blocks, row_seg, positions, part_acc,
                                               part_ml, n_chunks, scale, window, page_size, H, G, hd, 0, keep_first, front_slot0, 1)));
    return kp_launch_status();
}

// front_slot0: -1, or the slot from which the kept first keys' chunks lie (see kp_attention_front_chunks).
int kp_attention_merge_sink(const int* positions, void* out, int ldo, const float* scratch, int n_chunks,
                            int chunk_keys, int window, int block, int keep_first, const float* sink, int front_slot0, int n,
                            int H, int hd, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (hd < 16 || hd > KP_MAX_HEAD_DIM || n > 65535 || chunk_keys < 1) return KP_ERR_UNSUPPORTED;
    const float* part_acc = scratch;
    const float* part_ml = scratch + (size_t)n * H * n_chunks * hd;
    KP_DISPATCH_DTYPE(dtype, T, return launch_merge<T>(part_acc, part_ml, positions, out, ldo, n_chunks, chunk_keys, window,
                                                       block, keep_first, sink, n, H, hd, (cudaStream_t)stream, front_slot0));
    return kp_launch_status();
}

int kp_attention_merge_masked(const int* positions, void* out, int ldo, const float* scratch, int n_chunks,
                              int chunk_keys, int window, int block, int n, int H, int hd, int dtype, void* stream) {
    return kp_attention_merge_sink(positions, out, ldo, scratch, n_chunks, chunk_keys, window, block, 0, nullptr, -1, n, H, hd,
                                   dtype, stream);
}

int kp_attention_merge(const int* positions, void* out, int ldo, const float* scratch, int n_chunks, int chunk_keys,
                       int window, int n, int H, int hd, int dtype, void* stream) {
    return kp_attention_merge_masked(positions, out, ldo, scratch, n_chunks, chunk_keys, window, 0, n, H, hd, dtype, stream);
}

}  // extern "C"
