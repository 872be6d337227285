// Tensor-core flash attention (bfloat16, mma.sync m16n8k16) for prompts whose keys and values have sizes
// of their own: one build per pair (-DDFI_KEY_DIM=..., -DDFI_VALUE_DIM=..., multiples of 16 up to 256 and
// 128).  No rotation and no norm happen here: the queries come normalised, the cache holds the keys as
// they are scored.  A CTA of four warps takes 64 query rows of one (sequence, head); pages of 64 keys and
// values travel through a two-stage cp.async ring in padded shared memory; scores, the online softmax
// (log2 domain) and the weighted values stay in registers.  Before a row is stored it is multiplied by
// sigmoid(gate[row, head]) if gates are given, and by a constant: the head gate and a parallel mixer's
// weight cost no pass of their own.
#include "common.cuh"

#ifndef DFI_KEY_DIM
#define DFI_KEY_DIM 64
#endif
#ifndef DFI_VALUE_DIM
#define DFI_VALUE_DIM 64
#endif

namespace dfi {

constexpr int DK = DFI_KEY_DIM, DV = DFI_VALUE_DIM;
static_assert(DK % 16 == 0 && DK <= 256 && DV % 16 == 0 && DV <= 128, "sizes this kernel is built for");
constexpr int kPage = 64;
constexpr int kStrideK = DK + 8, kStrideV = DV + 8;   // padded rows: 16-byte chunks at an odd stride are conflict-free for ldmatrix
constexpr int kThreads = 128;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;   // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// One page of one head ([64][W], contiguous) into rows of W + 8; with `zero_dead`, rows whose key is not
// below `live_keys` are filled with zeros (values: what a masked weight of 0 multiplies must not be NaN).
template <int W>
__device__ __forceinline__ void load_page(bf16* dst, const bf16* src, int first_key, int live_keys, bool zero_dead) {
    constexpr int chunks = W / 8;
    for (int i = threadIdx.x; i < kPage * chunks; i += kThreads) {
        const int row = i / chunks, c = i % chunks;
        const bool valid = !zero_dead || first_key + row < live_keys;
        cp_async16(dst + row * (W + 8) + c * 8, src + (size_t)row * W + c * 8, valid);
    }
}

template <int W>
__device__ __forceinline__ const bf16* page_of(const bf16* cache, const int* table, int tile, int ring_tokens, int n_kv,
                                               int kv_head) {
    const int place = place_of(tile * kPage, ring_tokens);
    return cache + ((size_t)table[place / kPage] * n_kv + kv_head) * kPage * W;
}

__global__ void __launch_bounds__(kThreads)
attention_split_prefill_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                               const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                               const int* __restrict__ block_table, int table_width, const int* __restrict__ cu_rows,
                               const int* __restrict__ seq_start, int n_q, int n_kv, int ring_tokens, int window,
                               float scale_log2, const bf16* __restrict__ gate, int gate_stride, float out_scale) {
    pdl_launch_next();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);   // [64][kStrideK]
    bf16* k_s = q_s + kPage * kStrideK;              // [2][64][kStrideK]
    bf16* v_s = k_s + 2 * kPage * kStrideK;          // [2][64][kStrideV]

    const int seq = blockIdx.z, head = blockIdx.y;
    const int row0 = cu_rows[seq], q_len = cu_rows[seq + 1] - row0;
    const int r0 = blockIdx.x * 64;
    if (r0 >= q_len) return;
    const int rows_here = min(64, q_len - r0);
    const int start = seq_start[seq];
    const int kv_len = start + q_len;
    const int kv_head = head / (n_q / n_kv);
    const int* table = block_table + (size_t)seq * table_width;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int mi = lane >> 3, r = lane & 7;

    // the query tile; rows past the sequence's share are zeros
    for (int i = threadIdx.x; i < 64 * (DK / 8); i += kThreads) {
        const int row = i / (DK / 8), c = i % (DK / 8);
        const bool valid = row < rows_here;
        cp_async16(q_s + row * kStrideK + c * 8,
                   q + (size_t)(row0 + r0 + (valid ? row : 0)) * q_stride + (size_t)head * DK + c * 8, valid);
    }
    const int last_key = start + r0 + rows_here - 1;
    const int first_key = window > 0 ? max(0, start + r0 - window + 1) : 0;
    const int t_begin = first_key / kPage, t_end = last_key / kPage;
    load_page<DK>(k_s, page_of<DK>(k_cache, table, t_begin, ring_tokens, n_kv, kv_head), t_begin * kPage, kv_len, false);
    load_page<DV>(v_s, page_of<DV>(v_cache, table, t_begin, ring_tokens, n_kv, kv_head), t_begin * kPage, kv_len, true);
    cp_async_commit();

    uint32_t qf[DK / 16][4];
    float o[DV / 8][4];
#pragma unroll
    for (int n = 0; n < DV / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const int pos_lo = start + r0 + warp * 16 + g, pos_hi = pos_lo + 8;      // the two query rows a thread holds

    for (int t = t_begin; t <= t_end; ++t) {
        const int stage = (t - t_begin) & 1;
        if (t < t_end) {
            load_page<DK>(k_s + (stage ^ 1) * kPage * kStrideK, page_of<DK>(k_cache, table, t + 1, ring_tokens, n_kv, kv_head),
                          (t + 1) * kPage, kv_len, false);
            load_page<DV>(v_s + (stage ^ 1) * kPage * kStrideV, page_of<DV>(v_cache, table, t + 1, ring_tokens, n_kv, kv_head),
                          (t + 1) * kPage, kv_len, true);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (t == t_begin) {
#pragma unroll
            for (int kk = 0; kk < DK / 16; ++kk)
                ldmatrix_x4(qf[kk], q_s + (warp * 16 + r + (mi & 1) * 8) * kStrideK + kk * 16 + (mi >> 1) * 8);
        }
        const bf16* k_t = k_s + stage * kPage * kStrideK;
        const bf16* v_t = v_s + stage * kPage * kStrideV;
        // S [16 x 64] = Q [16 x DK] . K [64 x DK]^T
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk) {
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                uint32_t b[4];
                ldmatrix_x4(b, k_t + (j * 8 + r + (mi >> 1) * 8) * kStrideK + kk * 16 + (mi & 1) * 8);
                mma_bf16(s[j], qf[kk], b[0], b[1]);
                mma_bf16(s[j + 1], qf[kk], b[2], b[3]);
            }
        }
        const int key_base = t * kPage;
        // the tile needs masking if any of its keys is hidden from any row of this warp
        const bool partial = key_base + kPage - 1 > start + r0 + warp * 16 ||
                             (window > 0 && key_base < start + r0 + warp * 16 + 15 - window + 1);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = s[j][e] * scale_log2;
                if (partial) {
                    const int key = key_base + j * 8 + t4 * 2 + (e & 1);
                    const int pos = (e & 2) ? pos_hi : pos_lo;
                    v = (key <= pos && (window <= 0 || key > pos - window)) ? v : -INFINITY;
                }
                s[j][e] = v;
            }
        }
        // online softmax of the two rows (g, g + 8) this thread holds
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fmaxf(s[j][2 * h], s[j][2 * h + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m[h], mx);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;   // a row with nothing to see yet
            const float corr = exp2f(m[h] - m_use);
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                s[j][2 * h] = exp2f(s[j][2 * h] - m_use);
                s[j][2 * h + 1] = exp2f(s[j][2 * h + 1] - m_use);
                sum += s[j][2 * h] + s[j][2 * h + 1];
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            l[h] = l[h] * corr + sum;
            m[h] = m_new;
#pragma unroll
            for (int n = 0; n < DV / 8; ++n) {
                o[n][2 * h] *= corr;
                o[n][2 * h + 1] *= corr;
            }
        }
        // O [16 x DV] += P [16 x 64] . V [64 x DV]
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * c][0], s[2 * c][1]);
            a[1] = pack_bf16(s[2 * c][2], s[2 * c][3]);
            a[2] = pack_bf16(s[2 * c + 1][0], s[2 * c + 1][1]);
            a[3] = pack_bf16(s[2 * c + 1][2], s[2 * c + 1][3]);
#pragma unroll
            for (int n = 0; n < DV / 8; n += 2) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, v_t + (c * 16 + r + (mi & 1) * 8) * kStrideV + n * 8 + (mi >> 1) * 8);
                mma_bf16(o[n], a, b[0], b[1]);
                mma_bf16(o[n + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();   // everyone is done with this stage before the next load overwrites it
    }

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = warp * 16 + g + h * 8;
        if (row < rows_here) {
            float factor = l[h] > 0.f ? out_scale / l[h] : 0.f;
            if (gate != nullptr)
                factor /= 1.f + expf(-__bfloat162float(gate[(size_t)(row0 + r0 + row) * gate_stride + head]));
            bf16* dst = out + (size_t)(row0 + r0 + row) * out_stride + (size_t)head * DV;
#pragma unroll
            for (int n = 0; n < DV / 8; ++n) {
                // two neighbouring elements; the row's start may be 2-byte aligned only
                dst[n * 8 + t4 * 2] = __float2bfloat16_rn(o[n][2 * h] * factor);
                dst[n * 8 + t4 * 2 + 1] = __float2bfloat16_rn(o[n][2 * h + 1] * factor);
            }
        }
    }
}

constexpr int kSmemBytes = (3 * kPage * kStrideK + 2 * kPage * kStrideV) * (int)sizeof(bf16);

// ------------------------------------------------------------------ decode: one query row a sequence
// A CTA takes (sequence, key/value head, part): the part's share of the sequence's pages, for all query
// heads of the group at once: they are the (up to 16) rows of one m16n8k16 tile, so a page is read once
// for the whole group.  Pages travel through the same two-stage ring as above; each of the four warps
// scores 16 of a page's 64 keys and keeps its own running maximum, sum and weighted values; at the end the
// warps' results meet in shared memory and the part's result goes to `partial`
// [sequence, head, part, 2 + DV] (maximum in the log2 domain, sum, weighted values), which the merge
// kernel of the core library reduces, gates and scales (its maxima may be in any base as long as the
// parts agree in their unit: it is stored in natural units, as that kernel's own parts store it).
__global__ void __launch_bounds__(kThreads)
attention_split_decode_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ k_cache,
                              const bf16* __restrict__ v_cache, const int* __restrict__ block_table, int table_width,
                              const int* __restrict__ seq_start, int n_q, int n_kv, int ring_tokens, int window,
                              float scale_log2, int n_parts, float* __restrict__ partial) {
    pdl_launch_next();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);   // [16][kStrideK]
    bf16* k_s = q_s + 16 * kStrideK;                 // [2][64][kStrideK]
    bf16* v_s = k_s + 2 * kPage * kStrideK;          // [2][64][kStrideV]
    const int seq = blockIdx.x, kv_head = blockIdx.y, part = blockIdx.z;
    const int group = n_q / n_kv;
    const int pos = seq_start[seq];                  // the query's position; keys 0..pos are visible
    const int kv_len = pos + 1;
    const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
    const int page_lo = first_key / kPage, page_hi = pos / kPage;          // inclusive
    const int per = (page_hi - page_lo + 1 + n_parts - 1) / n_parts;
    const int t_begin = page_lo + part * per, t_end = min(page_hi, t_begin + per - 1);
    const int* table = block_table + (size_t)seq * table_width;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t4 = lane & 3, mi = lane >> 3, r = lane & 7;
    float* mine = partial + (((size_t)seq * n_q + (size_t)kv_head * group) * n_parts + part) * (size_t)(2 + DV);
    const size_t head_step = (size_t)n_parts * (2 + DV);
    if (t_begin > t_end) {                            // a part without pages: nothing seen
        for (int h = threadIdx.x; h < group; h += kThreads) {
            mine[h * head_step] = -INFINITY;
            mine[h * head_step + 1] = 0.f;
        }
        return;
    }
    for (int i = threadIdx.x; i < 16 * (DK / 8); i += kThreads) {
        const int row = i / (DK / 8), c = i % (DK / 8);
        const bool valid = row < group;
        cp_async16(q_s + row * kStrideK + c * 8,
                   q + (size_t)seq * q_stride + (size_t)(kv_head * group + (valid ? row : 0)) * DK + c * 8, valid);
    }
    load_page<DK>(k_s, page_of<DK>(k_cache, table, t_begin, ring_tokens, n_kv, kv_head), t_begin * kPage, kv_len, false);
    load_page<DV>(v_s, page_of<DV>(v_cache, table, t_begin, ring_tokens, n_kv, kv_head), t_begin * kPage, kv_len, true);
    cp_async_commit();

    uint32_t qf[DK / 16][4];
    float o[DV / 8][4];
#pragma unroll
    for (int n = 0; n < DV / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const int key0 = warp * 16;                       // this warp's keys of every page

    for (int t = t_begin; t <= t_end; ++t) {
        const int stage = (t - t_begin) & 1;
        if (t < t_end) {
            load_page<DK>(k_s + (stage ^ 1) * kPage * kStrideK, page_of<DK>(k_cache, table, t + 1, ring_tokens, n_kv, kv_head),
                          (t + 1) * kPage, kv_len, false);
            load_page<DV>(v_s + (stage ^ 1) * kPage * kStrideV, page_of<DV>(v_cache, table, t + 1, ring_tokens, n_kv, kv_head),
                          (t + 1) * kPage, kv_len, true);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (t == t_begin) {
#pragma unroll
            for (int kk = 0; kk < DK / 16; ++kk)
                ldmatrix_x4(qf[kk], q_s + (r + (mi & 1) * 8) * kStrideK + kk * 16 + (mi >> 1) * 8);
        }
        const bf16* k_t = k_s + stage * kPage * kStrideK;
        const bf16* v_t = v_s + stage * kPage * kStrideV;
        float s[2][4];
#pragma unroll
        for (int jj = 0; jj < 2; ++jj)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[jj][e] = 0.f;
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk) {
            uint32_t b[4];
            ldmatrix_x4(b, k_t + (key0 + r + (mi >> 1) * 8) * kStrideK + kk * 16 + (mi & 1) * 8);
            mma_bf16(s[0], qf[kk], b[0], b[1]);
            mma_bf16(s[1], qf[kk], b[2], b[3]);
        }
        const int key_base = t * kPage + key0;
#pragma unroll
        for (int jj = 0; jj < 2; ++jj)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key_base + jj * 8 + t4 * 2 + (e & 1);
                s[jj][e] = (key >= first_key && key <= pos) ? s[jj][e] * scale_log2 : -INFINITY;
            }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float mx = fmaxf(fmaxf(s[0][2 * h], s[0][2 * h + 1]), fmaxf(s[1][2 * h], s[1][2 * h + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m[h], mx);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float corr = exp2f(m[h] - m_use);
            float sum = 0.f;
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                s[jj][2 * h] = exp2f(s[jj][2 * h] - m_use);
                s[jj][2 * h + 1] = exp2f(s[jj][2 * h + 1] - m_use);
                sum += s[jj][2 * h] + s[jj][2 * h + 1];
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            l[h] = l[h] * corr + sum;
            m[h] = m_new;
#pragma unroll
            for (int n = 0; n < DV / 8; ++n) {
                o[n][2 * h] *= corr;
                o[n][2 * h + 1] *= corr;
            }
        }
        uint32_t a[4];
        a[0] = pack_bf16(s[0][0], s[0][1]);
        a[1] = pack_bf16(s[0][2], s[0][3]);
        a[2] = pack_bf16(s[1][0], s[1][1]);
        a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int n = 0; n < DV / 8; n += 2) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, v_t + (key0 + r + (mi & 1) * 8) * kStrideV + n * 8 + (mi >> 1) * 8);
            mma_bf16(o[n], a, b[0], b[1]);
            mma_bf16(o[n + 1], a, b[2], b[3]);
        }
        __syncthreads();
    }
    // the four warps' results meet in shared memory (the ring is free now)
    float* m_s = reinterpret_cast<float*>(smem_raw);          // [4][16]
    float* l_s = m_s + 64;                                     // [4][16]
    float* o_s = l_s + 64;                                     // [4][16][DV]
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = g + h * 8;
        if (t4 == 0) { m_s[warp * 16 + row] = m[h]; l_s[warp * 16 + row] = l[h]; }
#pragma unroll
        for (int n = 0; n < DV / 8; ++n) {
            o_s[(warp * 16 + row) * DV + n * 8 + t4 * 2] = o[n][2 * h];
            o_s[(warp * 16 + row) * DV + n * 8 + t4 * 2 + 1] = o[n][2 * h + 1];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < group * DV; i += kThreads) {
        const int row = i / DV, d = i - row * DV;
        float m_all = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m_all = fmaxf(m_all, m_s[w * 16 + row]);
        float v = 0.f, l_all = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = m_s[w * 16 + row];
            if (mw != -INFINITY) {
                const float c = exp2f(mw - m_all);
                v += o_s[(w * 16 + row) * DV + d] * c;
                l_all += l_s[w * 16 + row] * c;
            }
        }
        float* dst = mine + row * head_step;
        if (d == 0) {
            dst[0] = m_all == -INFINITY ? -INFINITY : m_all * 0.6931471805599453f;   // natural units for the merge
            dst[1] = l_all;
        }
        dst[2 + d] = v;
    }
}

constexpr int kDecodeRing = (16 * kStrideK + 2 * kPage * kStrideK + 2 * kPage * kStrideV) * (int)sizeof(bf16);
constexpr int kDecodeMerge = (128 + 4 * 16 * DV) * (int)sizeof(float);
constexpr int kDecodeSmemBytes = kDecodeRing > kDecodeMerge ? kDecodeRing : kDecodeMerge;

}  // namespace dfi

using namespace dfi;

DFI_EXPORT int dfi_attention_split_set_pdl(int enabled) {
    const int before = pdl_enabled();
    pdl_enabled() = enabled ? 1 : 0;
    return before;
}

DFI_EXPORT int dfi_attention_split_key_dim() { return DK; }
DFI_EXPORT int dfi_attention_split_value_dim() { return DV; }

// q [rows, q_stride]: n_q heads of DK per row, normalised; out [rows, out_stride]: n_q heads of DV.
// cu_rows / seq_start [n_seqs (+1)]: the packed rows of each sequence and the position of its first row.
// gate (or null) [rows, gate_stride]: one number per row and head.  q rows and the caches 16-byte aligned.
DFI_EXPORT int dfi_attention_split_prefill(const void* q, int q_stride, void* out, int out_stride, const void* k_cache,
                                           const void* v_cache, const int* block_table, int table_width,
                                           const int* cu_rows, const int* seq_start, int n_seqs, int max_q_len, int n_q,
                                           int n_kv, int page_size, int ring_tokens, int window, float scale,
                                           const void* gate, int gate_stride, float out_scale, void* stream) {
    if (n_seqs <= 0 || max_q_len <= 0) return DFI_OK;
    if (page_size != kPage || n_q <= 0 || n_kv <= 0 || n_q % n_kv || table_width <= 0) return DFI_ERR_SHAPE;
    if (n_q > 65535 || n_seqs > 65535) return DFI_ERR_LIMIT;
    if (!aligned16(q) || q_stride % 8 || !aligned16(k_cache) || !aligned16(v_cache)) return DFI_ERR_ALIGN;
    static bool raised = false;
    if (!raised) {
        if (cudaFuncSetAttribute(attention_split_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) {
            cudaGetLastError();
            return DFI_ERR_LAUNCH;
        }
        raised = true;
    }
    dim3 grid((max_q_len + 63) / 64, n_q, n_seqs);
    launch(attention_split_prefill_kernel, grid, dim3(kThreads), (size_t)kSmemBytes, (cudaStream_t)stream, (const bf16*)q,
           q_stride, (bf16*)out, out_stride, (const bf16*)k_cache, (const bf16*)v_cache, block_table, table_width, cu_rows,
           seq_start, n_q, n_kv, ring_tokens, window, scale * kLog2e, (const bf16*)gate, gate_stride, out_scale);
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

// One query row per sequence (row i is sequence i, at position seq_start[i], its key and value already in
// the cache), at most 16 query heads per key/value head.  Writes `partial` [n_seqs, n_q, n_parts, 2 + DV]
// float32 for the merge kernel (dfi_split_merge of the core library).
DFI_EXPORT int dfi_attention_split_decode(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                          const int* block_table, int table_width, const int* seq_start, int n_seqs,
                                          int n_q, int n_kv, int page_size, int ring_tokens, int window, float scale,
                                          int n_parts, float* partial, void* stream) {
    if (n_seqs <= 0) return DFI_OK;
    if (page_size != kPage || n_q <= 0 || n_kv <= 0 || n_q % n_kv || n_q / n_kv > 16 || table_width <= 0) return DFI_ERR_SHAPE;
    if (n_parts <= 0 || n_parts > 65535 || n_kv > 65535 || partial == nullptr) return DFI_ERR_SHAPE;
    if (!aligned16(q) || q_stride % 8 || !aligned16(k_cache) || !aligned16(v_cache)) return DFI_ERR_ALIGN;
    static bool raised = false;
    if (!raised) {
        if (cudaFuncSetAttribute(attention_split_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecodeSmemBytes) != cudaSuccess) {
            cudaGetLastError();
            return DFI_ERR_LAUNCH;
        }
        raised = true;
    }
    launch(attention_split_decode_kernel, dim3(n_seqs, n_kv, n_parts), dim3(kThreads), (size_t)kDecodeSmemBytes,
           (cudaStream_t)stream, (const bf16*)q, q_stride, (const bf16*)k_cache, (const bf16*)v_cache, block_table,
           table_width, seq_start, n_q, n_kv, ring_tokens, window, scale * kLog2e, n_parts, partial);
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}
