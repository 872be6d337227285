// Attention whose values have a size of their own (key size D, value size DV), without rotation:
// the per-head norm of queries and keys with the cache write, and the decode step's attention dealt
// over the keys of every sequence.
//
// Row layout of the projection that both kernels read: n_q query heads of D, n_kv key heads of D,
// n_kv value heads of DV (anything after that, gates for instance, is the caller's).
#include "common.cuh"

namespace dfi {

constexpr int kNormWarps = 4;

// One warp per (row, head slot): query heads are normalised in place, key heads normalised into the key
// cache, value heads copied into the value cache.  The norm is x / sqrt(mean(x^2) + eps) * w with w
// shared by all heads (q_w, k_w float32 [D]; null: no norm).  Any D and DV: a lane takes elements
// lane, lane + 32, ...
template <typename T>
__global__ void head_norm_write_kernel(T* __restrict__ proj, int row_stride, int n_q, int n_kv, int D, int DV,
                                       const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                       const int* __restrict__ row_pos, const int* __restrict__ row_seq,
                                       T* __restrict__ k_cache, T* __restrict__ v_cache,
                                       const int* __restrict__ block_table, int table_width, int page_size,
                                       int ring_tokens, int write_cache) {
    pdl_launch_next();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int slot = blockIdx.y * kNormWarps + (threadIdx.x >> 5);
    if (slot >= n_q + 2 * n_kv) return;
    const int row = blockIdx.x;
    const bool is_q = slot < n_q, is_k = !is_q && slot < n_q + n_kv;
    if (!is_q && !write_cache) return;
    const int size = is_q || is_k ? D : DV;
    T* src = proj + (size_t)row * row_stride +
             (is_q ? (size_t)slot * D : is_k ? (size_t)slot * D : (size_t)(n_q + n_kv) * D + (size_t)(slot - n_q - n_kv) * DV);
    T* dst = src;
    if (!is_q) {
        const int place = place_of(row_pos[row], ring_tokens);
        const int page = block_table[(size_t)row_seq[row] * table_width + place / page_size];
        const int kv_head = is_k ? slot - n_q : slot - n_q - n_kv;
        dst = (is_k ? k_cache : v_cache) + (((size_t)page * n_kv + kv_head) * page_size + place % page_size) * size;
    }
    const float* w = is_q ? q_w : (is_k ? k_w : nullptr);
    float factor = 1.f;
    if (w != nullptr) {
        float ssq = 0.f;
        for (int i = lane; i < size; i += 32) {
            const float v = to_float(src[i]);
            ssq += v * v;
        }
        ssq = warp_sum(ssq);
        factor = 1.0f / sqrtf(ssq / (float)size + eps);
    }
    for (int i = lane; i < size; i += 32) {
        float v = to_float(src[i]);
        if (w != nullptr) v = v * factor * w[i];
        dst[i] = from_float<T>(v);
    }
}

// ------------------------------------------------------------------ decode: one query row a sequence
// A CTA of kSplitWarps warps takes (sequence, key/value head, part): the part's share of the sequence's
// keys, for all query heads of the group, one query head after another (the keys stay in L1/L2 between
// them).  Every warp runs the online softmax over its keys (32 at a time, one a lane); the warps' results
// meet in shared memory, the parts' in `partial` [seq, head, part, 2 + DV] (max, sum, weighted values),
// which the merge kernel below reduces, gates and scales.
constexpr int kSplitWarps = 4;
constexpr int kSplitMaxDim = 256;

template <typename T>
__global__ void split_decode_kernel(const T* __restrict__ q, int q_row_stride, const T* __restrict__ k_cache,
                                    const T* __restrict__ v_cache, const int* __restrict__ block_table,
                                    int table_width, const int* __restrict__ seq_start, int n_q, int n_kv, int D,
                                    int DV, int page_size, int ring_tokens, int window, float scale, int n_parts,
                                    float* __restrict__ partial) {
    pdl_launch_next();
    pdl_wait();
    __shared__ float q_s[kSplitMaxDim];
    __shared__ float m_s[kSplitWarps], l_s[kSplitWarps];
    __shared__ float acc_s[kSplitWarps][kSplitMaxDim];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int seq = blockIdx.x, kv_head = blockIdx.y, part = blockIdx.z;
    const int group = n_q / n_kv;
    const int pos = seq_start[seq];                       // the query's position: keys 0..pos are visible
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    const int n_keys = pos - first + 1;
    // whole tiles of 32 keys per part, so that parts do not share a tile
    const int tiles = (n_keys + 31) / 32, per = (tiles + n_parts - 1) / n_parts;
    const int lo = first + part * per * 32, hi = min(pos + 1, lo + per * 32);
    const int* table = block_table + (size_t)seq * table_width;

    for (int g = 0; g < group; ++g) {
        const int head = kv_head * group + g;
        __syncthreads();
        for (int d = threadIdx.x; d < D; d += blockDim.x)
            q_s[d] = to_float(q[(size_t)seq * q_row_stride + (size_t)head * D + d]) * scale;
        __syncthreads();
        float acc[kSplitMaxDim / 32];
#pragma unroll
        for (int j = 0; j < kSplitMaxDim / 32; ++j) acc[j] = 0.f;
        float m = -INFINITY, l = 0.f;
        for (int base = lo + warp * 32; base < hi; base += kSplitWarps * 32) {
            const int key = base + lane;
            const bool live = key < hi;
            unsigned long long offset = 0;
            float s = -INFINITY;
            if (live) {
                const int place = place_of(key, ring_tokens);
                offset = ((unsigned long long)table[place / page_size] * n_kv + kv_head) * page_size + place % page_size;
                const T* kp = k_cache + offset * D;
                float dot = 0.f;
                for (int d = 0; d < D; ++d) dot += q_s[d] * to_float(kp[d]);
                s = dot;
            }
            const float m_new = fmaxf(m, warp_max(s));
            const float corr = expf(m - m_new);
            const float p = live ? expf(s - m_new) : 0.f;
            l = l * corr + warp_sum(p);
#pragma unroll
            for (int j = 0; j < kSplitMaxDim / 32; ++j) acc[j] *= corr;
            m = m_new;
            const int count = min(32, hi - base);
            for (int kk = 0; kk < count; ++kk) {
                const float pk = __shfl_sync(0xffffffffu, p, kk);
                const unsigned long long off = __shfl_sync(0xffffffffu, offset, kk);
                const T* vp = v_cache + off * DV;
#pragma unroll
                for (int j = 0; j < kSplitMaxDim / 32; ++j) {
                    const int d = lane + 32 * j;
                    if (d < DV) acc[j] += pk * to_float(vp[d]);
                }
            }
        }
        if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
        for (int j = 0; j < kSplitMaxDim / 32; ++j) {
            const int d = lane + 32 * j;
            if (d < DV) acc_s[warp][d] = acc[j];
        }
        __syncthreads();
        float m_all = -INFINITY;
#pragma unroll
        for (int w = 0; w < kSplitWarps; ++w) m_all = fmaxf(m_all, m_s[w]);
        float* dst = partial + (((size_t)seq * n_q + head) * n_parts + part) * (size_t)(2 + DV);
        float l_all = 0.f;
#pragma unroll
        for (int w = 0; w < kSplitWarps; ++w) l_all += m_s[w] == -INFINITY ? 0.f : l_s[w] * expf(m_s[w] - m_all);
        if (threadIdx.x == 0) { dst[0] = m_all; dst[1] = l_all; }
        for (int d = threadIdx.x; d < DV; d += blockDim.x) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < kSplitWarps; ++w)
                if (m_s[w] != -INFINITY) v += acc_s[w][d] * expf(m_s[w] - m_all);
            dst[2 + d] = v;
        }
    }
}

// One warp per (sequence, query head): merges the parts, applies sigmoid(gate) and out_scale.  Lane p first
// works out part p's weight exp(m_p - m) (parts beyond 32 in rounds), then every lane sums its columns over
// the parts with the loads of eight parts in flight at once.
template <typename T>
__global__ void split_merge_kernel(const float* __restrict__ partial, int n_q, int DV, int n_parts,
                                   const T* __restrict__ gate, int gate_row_stride, float out_scale,
                                   T* __restrict__ out, int out_row_stride) {
    pdl_launch_next();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5), seq = blockIdx.x;
    if (head >= n_q) return;
    const size_t stride = (size_t)(2 + DV);
    const float* src = partial + ((size_t)seq * n_q + head) * n_parts * stride;
    float m = -INFINITY;
    for (int p = lane; p < n_parts; p += 32) m = fmaxf(m, src[p * stride]);
    m = warp_max(m);
    float l = 0.f;
    for (int p = lane; p < n_parts; p += 32) {
        const float mp = src[p * stride];
        if (mp != -INFINITY) l += src[p * stride + 1] * expf(mp - m);
    }
    l = warp_sum(l);
    float factor = out_scale / l;
    if (gate != nullptr) factor /= 1.f + expf(-to_float(gate[(size_t)seq * gate_row_stride + head]));
    float acc[8];                                    // columns lane, lane + 32, ... (DV <= 256)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int p0 = 0; p0 < n_parts; p0 += 32) {
        const int mine = p0 + lane;
        const float mp = mine < n_parts ? src[mine * stride] : -INFINITY;
        const float weight = mp == -INFINITY ? 0.f : expf(mp - m);
        const int count = min(32, n_parts - p0);
        // every load is issued whatever its index (clamped): a straight run of loads whose latencies overlap;
        // a part or a column that does not exist gets the weight 0
        const int n_cols = (DV + 31) >> 5;
        for (int pp = 0; pp < 32; pp += 4) {
            if (pp >= count) break;
            float c[4], x[4][8];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                c[u] = pp + u < count ? __shfl_sync(0xffffffffu, weight, (pp + u) & 31) : 0.f;
                const float* row = src + (size_t)(p0 + min(pp + u, count - 1)) * stride + 2;
#pragma unroll
                for (int j = 0; j < 8; ++j) x[u][j] = j < n_cols ? __ldg(row + min(lane + 32 * j, DV - 1)) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = fmaf(c[u], x[u][j], acc[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int d = lane + 32 * j;
        if (d < DV) out[(size_t)seq * out_row_stride + (size_t)head * DV + d] = from_float<T>(acc[j] * factor);
    }
}

}  // namespace dfi

using namespace dfi;

DFI_EXPORT int dfi_head_norm_write(void* proj, int rows, int row_stride, int n_q, int n_kv, int head_dim, int v_dim,
                                   const float* q_w, const float* k_w, float eps, const int* row_pos,
                                   const int* row_seq, void* k_cache, void* v_cache, const int* block_table,
                                   int table_width, int page_size, int ring_tokens, int write_cache, int dtype,
                                   void* stream) {
    if (rows <= 0) return DFI_OK;
    if (head_dim <= 0 || v_dim <= 0 || n_q <= 0 || n_kv <= 0 || page_size <= 0 || table_width <= 0) return DFI_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid(rows, (n_q + 2 * n_kv + kNormWarps - 1) / kNormWarps);
    if (grid.y > 65535) return DFI_ERR_LIMIT;
    if (dtype == DFI_DTYPE_F32)
        launch(head_norm_write_kernel<float>, grid, kNormWarps * 32, 0, st, (float*)proj, row_stride, n_q, n_kv, head_dim,
               v_dim, q_w, k_w, eps, row_pos, row_seq, (float*)k_cache, (float*)v_cache, block_table, table_width,
               page_size, ring_tokens, write_cache);
    else if (dtype == DFI_DTYPE_BF16)
        launch(head_norm_write_kernel<bf16>, grid, kNormWarps * 32, 0, st, (bf16*)proj, row_stride, n_q, n_kv, head_dim,
               v_dim, q_w, k_w, eps, row_pos, row_seq, (bf16*)k_cache, (bf16*)v_cache, block_table, table_width,
               page_size, ring_tokens, write_cache);
    else return DFI_ERR_DTYPE;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

// floats of scratch that dfi_split_decode needs
DFI_EXPORT long long dfi_split_decode_floats(int n_seqs, int n_q, int v_dim, int n_parts) {
    return (long long)n_seqs * n_q * n_parts * (2 + v_dim);
}

// One query row per sequence (row i belongs to sequence i and sits at position seq_start[i], its key and
// value already in the cache).  q [n_seqs, q_row_stride]; out [n_seqs, out_row_stride] n_q heads of v_dim.
DFI_EXPORT int dfi_split_decode(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_cache,
                                const void* v_cache, const int* block_table, int table_width, const int* seq_start,
                                int n_seqs, int n_q, int n_kv, int head_dim, int v_dim, int page_size,
                                int ring_tokens, int window, float scale, const void* gate, int gate_row_stride,
                                float out_scale, int n_parts, float* partial, int dtype, void* stream) {
    if (n_seqs <= 0) return DFI_OK;
    if (head_dim <= 0 || head_dim > kSplitMaxDim || v_dim <= 0 || v_dim > kSplitMaxDim) return DFI_ERR_SHAPE;
    if (n_q <= 0 || n_kv <= 0 || n_q % n_kv || n_parts <= 0 || n_parts > 65535 || n_kv > 65535) return DFI_ERR_SHAPE;
    if (partial == nullptr) return DFI_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid(n_seqs, n_kv, n_parts), merge_grid(n_seqs, (n_q + 3) / 4);
    if (dtype == DFI_DTYPE_F32) {
        launch(split_decode_kernel<float>, grid, kSplitWarps * 32, 0, st, (const float*)q, q_row_stride,
               (const float*)k_cache, (const float*)v_cache, block_table, table_width, seq_start, n_q, n_kv, head_dim,
               v_dim, page_size, ring_tokens, window, scale, n_parts, partial);
        launch(split_merge_kernel<float>, merge_grid, 128, 0, st, (const float*)partial, n_q, v_dim, n_parts,
               (const float*)gate, gate_row_stride, out_scale, (float*)out, out_row_stride);
    } else if (dtype == DFI_DTYPE_BF16) {
        launch(split_decode_kernel<bf16>, grid, kSplitWarps * 32, 0, st, (const bf16*)q, q_row_stride,
               (const bf16*)k_cache, (const bf16*)v_cache, block_table, table_width, seq_start, n_q, n_kv, head_dim,
               v_dim, page_size, ring_tokens, window, scale, n_parts, partial);
        launch(split_merge_kernel<bf16>, merge_grid, 128, 0, st, (const float*)partial, n_q, v_dim, n_parts,
               (const bf16*)gate, gate_row_stride, out_scale, (bf16*)out, out_row_stride);
    } else return DFI_ERR_DTYPE;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

// The merge alone: `partial` [n_seqs, n_q, n_parts, 2 + v_dim] (maximum in natural units, sum, weighted
// values) as some other kernel left it; out [n_seqs, out_row_stride] in `dtype`, gated and scaled.
DFI_EXPORT int dfi_split_merge(const float* partial, int n_seqs, int n_q, int v_dim, int n_parts, const void* gate,
                               int gate_row_stride, float out_scale, void* out, int out_row_stride, int dtype,
                               void* stream) {
    if (n_seqs <= 0) return DFI_OK;
    if (n_q <= 0 || v_dim <= 0 || n_parts <= 0 || partial == nullptr) return DFI_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid(n_seqs, (n_q + 3) / 4);
    if (dtype == DFI_DTYPE_F32)
        launch(split_merge_kernel<float>, grid, 128, 0, st, partial, n_q, v_dim, n_parts, (const float*)gate,
               gate_row_stride, out_scale, (float*)out, out_row_stride);
    else if (dtype == DFI_DTYPE_BF16)
        launch(split_merge_kernel<bf16>, grid, 128, 0, st, partial, n_q, v_dim, n_parts, (const bf16*)gate,
               gate_row_stride, out_scale, (bf16*)out, out_row_stride);
    else return DFI_ERR_DTYPE;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}
