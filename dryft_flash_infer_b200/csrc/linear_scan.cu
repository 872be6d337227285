// Mixers with a matrix state per head: S [D, V] float32 per (sequence, head), carried from token to
// token, decayed per key channel.  Two orders of the same recurrence:
//
//   decay-then-read   S_t = diag(a_t) S_(t-1) + k_t v_t^T ;  o_t = S_t^T q_t
//                     a = sigmoid(z)^(1/tau)                             (gated linear attention)
//   read-then-decay   o_t = (S_(t-1) + diag(u) k_t v_t^T)^T q_t ;  S_t = diag(a_t) S_(t-1) + k_t v_t^T
//                     a = exp(-exp(z))                                   (RWKV-style time mixing)
//
// where z = decay_logit + decay_bias is float32.  State, decays, their logarithms and exponentials and the
// reads are float32 whatever the storage type of q, k, v; the recurrence runs in the order of the tokens,
// so a prompt taken whole, in portions or token by token gives the same state up to nothing at all.
//
// One CTA of eight warps owns one (sequence, head, 32 or 16 columns of S) for all the tokens the step brings
// it: a column of S needs no other column, so a head spreads over V / 32 (or V / 16) CTAs.  Warp w keeps rows
// [w NI, (w+1) NI) of its columns in registers, lane c column c.  Tokens are fetched up to 64 at a time: their
// q, k, decays and v wait in shared memory as float32 (the decay computed once per token and channel), and
// while they are worked through the next ones are already on their way from global memory into registers:
// with few CTAs per SM the latency of those loads, not the arithmetic, is what a token costs, so a fetch
// has to cover many tokens.  Every warp leaves its rows' share of o_t in shared memory; after every
// sixteen tokens the shares are summed and stored as float32.  A second kernel, one warp per (row, head), divides a head's
// output by its root mean square, weights it, gates it with silu(g) and stores it in the storage type.
//
// The token shift of the time-mixing layer (every projection reads its own blend of a token's row and
// the row before it) is the other kernel here; the row that a sequence's next step will need lives in
// the same state area as S and is written by the scan kernel, which runs after the blends were read.
#include "common.cuh"

namespace dfi {

constexpr int kScanWarps = 8;
constexpr int kScanTokens = 16;     // tokens staged in shared memory at a time

struct ScanArgs {
    const void* q; const void* k; const void* v; const void* g;       // [rows, *_stride] in the storage type
    int q_stride, k_stride, v_stride, g_stride;
    const float* decay_logit;      // [rows, H * D]
    const float* decay_bias;       // [H * D] or null
    const float* bonus;            // [H * D] (read-then-decay only)
    float decay_param;             // tau
    float q_scale;
    float* state;                  // [slots, slot_stride]; a slot holds S [H, D, V] first
    long long slot_stride;
    const int* cu_rows;            // [sequences + 1]
    const int* seq_slot;           // [sequences]
    int H, D, V;
    float* raw;                    // [rows, H * V]: the reads o_t before norm and gate
    const void* carry_rows;        // or null: [rows, carry_width] rows whose last one per sequence is kept in the state
    int carry_width;
    long long carry_offset;        // where in a slot that row lives
    int bf16;                      // storage type of q, k, v, g, out, carry_rows
};

// Through the read-only path (ld.global.nc): the rows are written by earlier kernels only, and a load that
// cannot alias shared memory may be issued ahead of the stores into it.
__device__ __forceinline__ float load_as_float(const void* p, size_t i, int is_bf16) {
    if (is_bf16) {
        const unsigned short raw = __ldg(reinterpret_cast<const unsigned short*>(p) + i);
        return __uint_as_float((unsigned int)raw << 16);
    }
    return __ldg(reinterpret_cast<const float*>(p) + i);
}
__device__ __forceinline__ void store_from_float(void* p, size_t i, float v, int is_bf16) {
    if (is_bf16) reinterpret_cast<bf16*>(p)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<float*>(p)[i] = v;
}

template <int MODE>
__device__ __forceinline__ float decay_of(float z, float param) {
    if (MODE == 0) {
        // sigmoid(z)^(1/tau) = exp(-softplus(-z) / tau)
        const float sp = fmaxf(-z, 0.f) + log1pf(expf(-fabsf(z)));
        return expf(-sp / param);
    }
    return expf(-expf(z));
}

// Tokens per fetch of a prompt's rows: as many as shared memory and the registers of the fetch allow while
// two CTAs still fit an SM for the narrow heads.  Steps of at most 16 rows a sequence (decoding, short
// portions) fetch 16: few registers, so that many (sequence, head) pairs run at once.
__host__ __device__ constexpr int scan_fetch_tokens(int ni) { return ni <= 16 ? 32 : 16; }

// What a thread fetches for the chunk of up to TC tokens at row c0: elements tid, tid + THREADS, ... of
// [TC][DP] (q, k, decay logits) and of [TC][COLS] (v, the CTA's columns from col0 on).
template <typename T, int TC, int DP, int COLS, int PER, int PER_V>
__device__ __forceinline__ void scan_fetch(const ScanArgs& a, int c0, int row1, int head, int col0, int tid,
                                           T (&fq)[PER], T (&fk)[PER], float (&fz)[PER], T (&fv)[PER_V]) {
    // Every load is issued whatever its index (clamped into the chunk and the head) and nothing is done with
    // its value here: one straight run of loads, whose latencies overlap; what lies outside is set to zero
    // when the values are moved to shared memory.
    constexpr int THREADS = kScanWarps * 32;
    const int last = min(TC, row1 - c0) - 1, D = a.D, V = a.V, HD = a.H * a.D;
    const T* q = reinterpret_cast<const T*>(a.q);
    const T* k = reinterpret_cast<const T*>(a.k);
    const T* v = reinterpret_cast<const T*>(a.v);
#pragma unroll
    for (int e = 0; e < PER; ++e) {
        const int idx = tid + e * THREADS, t = min(idx / DP, last), i = min(idx % DP, D - 1);
        const size_t row = (size_t)(c0 + t);
        const int col = head * D + i;
        fq[e] = __ldg(q + row * a.q_stride + col);
        fk[e] = __ldg(k + row * a.k_stride + col);
        fz[e] = __ldg(a.decay_logit + row * HD + col);
    }
#pragma unroll
    for (int e = 0; e < PER_V; ++e) {
        const int idx = tid + e * THREADS, t = min(idx / COLS, last);
        fv[e] = __ldg(v + (size_t)(c0 + t) * a.v_stride + head * V + min(col0 + idx % COLS, V - 1));
    }
}

// COLS: columns of S per CTA, 32 (a lane a column) or 16: then the two halves of a warp share the columns and
// split the warp's rows, their shares of o_t meet by one shuffle, and a head spreads over twice the CTAs (for
// steps with fewer (sequence, head, 32 columns) than SMs).
template <typename T, int MODE, int NI, int TC, int COLS>
__global__ void __launch_bounds__(kScanWarps * 32, (NI <= 8 ? 2 : 1)) linear_scan_kernel(const ScanArgs a) {
    constexpr int DP = kScanWarps * NI, THREADS = kScanWarps * 32;
    constexpr int NIL = NI * COLS / 32;               // rows of S a lane keeps
    static_assert(NIL % 4 == 0, "a lane's rows come in fours");
    constexpr int PER = TC * DP / THREADS;            // elements of q, k, z a thread fetches per chunk
    constexpr int PER_V = TC * COLS / THREADS;        // and of v
    static_assert(PER_V >= 1, "every thread fetches a value");
    extern __shared__ __align__(16) float smem[];
    float* rs = smem;                                 // [TC][DP]
    float* ks = rs + TC * DP;                         // [TC][DP]
    float* ws = ks + TC * DP;                         // [TC][DP]
    float* vs = ws + TC * DP;                         // [TC][COLS]
    float* op = vs + TC * COLS;                       // [kScanTokens][warps][COLS]
    pdl_launch_next();
    pdl_wait();
    const int seq = blockIdx.x, head = blockIdx.y;
    const int row0 = a.cu_rows[seq], row1 = a.cu_rows[seq + 1];
    if (row1 <= row0) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int D = a.D, V = a.V;
    const int col0 = blockIdx.z * COLS, cl = lane % COLS;
    const int j = col0 + cl;                          // this lane's column of S
    float* S_g = a.state + (size_t)a.seq_slot[seq] * a.slot_stride + (size_t)head * D * V;
    const int i0 = warp * NI + (lane / COLS) * NIL;   // and the first of its rows

    float S[NIL], U[NIL];
#pragma unroll
    for (int n = 0; n < NIL; ++n) {
        const int i = i0 + n;
        U[n] = (MODE == 1 && i < D) ? a.bonus[head * D + i] : 0.f;
        S[n] = (i < D && j < V) ? S_g[(size_t)i * V + j] : 0.f;
    }

    T fq[PER], fk[PER], fv[PER_V];
    float fz[PER];
    float bias[PER];
#pragma unroll
    for (int e = 0; e < PER; ++e) {
        const int i = (tid + e * THREADS) % DP;
        bias[e] = (a.decay_bias != nullptr && i < D) ? a.decay_bias[head * D + i] : 0.f;
    }

    scan_fetch<T, TC, DP, COLS, PER, PER_V>(a, row0, row1, head, col0, tid, fq, fk, fz, fv);
    for (int c0 = row0; c0 < row1; c0 += TC) {
        const int nt = min(TC, row1 - c0);
        __syncthreads();                               // the chunk before is done with shared memory
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            const int idx = tid + e * THREADS, i = idx % DP;
            const bool live = i < D && idx / DP < nt;
            rs[idx] = live ? to_float(fq[e]) * a.q_scale : 0.f;
            ks[idx] = live ? to_float(fk[e]) : 0.f;
            ws[idx] = live ? decay_of<MODE>(fz[e] + bias[e], a.decay_param) : 1.f;
        }
#pragma unroll
        for (int e = 0; e < PER_V; ++e) {
            const int idx = tid + e * THREADS;
            vs[idx] = (col0 + idx % COLS < V && idx / COLS < nt) ? to_float(fv[e]) : 0.f;
        }
        __syncthreads();
        if (c0 + TC < row1)                            // on its way while this chunk is worked through
            scan_fetch<T, TC, DP, COLS, PER, PER_V>(a, c0 + TC, row1, head, col0, tid, fq, fk, fz, fv);
        for (int s0 = 0; s0 < nt; s0 += kScanTokens) {
            const int ns = min(kScanTokens, nt - s0);
#pragma unroll 2
            for (int t = s0; t < s0 + ns; ++t) {
                const float vj = vs[t * COLS + cl];
                float o = 0.f;
                const float4* r4 = reinterpret_cast<const float4*>(rs + t * DP + i0);
                const float4* k4 = reinterpret_cast<const float4*>(ks + t * DP + i0);
                const float4* w4 = reinterpret_cast<const float4*>(ws + t * DP + i0);
#pragma unroll
                for (int n4 = 0; n4 < NIL / 4; ++n4) {
                    const float4 rv = r4[n4], kv4 = k4[n4], wv = w4[n4];
                    const float r[4] = {rv.x, rv.y, rv.z, rv.w}, k[4] = {kv4.x, kv4.y, kv4.z, kv4.w}, w[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int n = n4 * 4 + e;
                        if (MODE == 0) {
                            S[n] = fmaf(w[e], S[n], k[e] * vj);
                            o = fmaf(r[e], S[n], o);
                        } else {
                            const float kv = k[e] * vj;
                            o = fmaf(r[e], fmaf(U[n], kv, S[n]), o);
                            S[n] = fmaf(w[e], S[n], kv);
                        }
                    }
                }
                if (COLS < 32) o += __shfl_xor_sync(0xffffffffu, o, COLS);
                if (lane < COLS) op[((t - s0) * kScanWarps + warp) * COLS + lane] = o;
            }
            __syncthreads();
            // sixteen tokens' reads: the warps' shares summed, float32, a row's 32 columns side by side
            for (int t = warp; t < ns; t += kScanWarps) {
                float sum = 0.f;
#pragma unroll
                for (int w8 = 0; w8 < kScanWarps; ++w8) sum += op[(t * kScanWarps + w8) * COLS + cl];
                if (lane < COLS && j < V) a.raw[(size_t)(c0 + s0 + t) * (a.H * V) + head * V + j] = sum;
            }
            __syncthreads();
        }
    }
#pragma unroll
    for (int n = 0; n < NIL; ++n) {
        const int i = i0 + n;
        if (i < D && j < V) S_g[(size_t)i * V + j] = S[n];
    }
    if (a.carry_rows != nullptr && head == 0 && blockIdx.z == 0) {
        float* dst = a.state + (size_t)a.seq_slot[seq] * a.slot_stride + a.carry_offset;
        for (int c = tid; c < a.carry_width; c += THREADS)
            dst[c] = load_as_float(a.carry_rows, (size_t)(row1 - 1) * a.carry_width + c, a.bf16);
    }
}

// out[row, head] = raw[row, head] / rms(raw[row, head]) * weight * silu(g[row, head]) * out_scale: one warp per
// (row, head); weight [V] (norm_head_stride 0) or [H, V] (norm_head_stride V) or null; g null: no gate.
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ raw, int H, int V, const float* __restrict__ weight,
                                      int norm_head_stride, float eps, const T* __restrict__ g, int g_stride,
                                      float out_scale, T* __restrict__ out, int out_stride) {
    pdl_launch_next();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (head >= H) return;
    const size_t row = blockIdx.x;
    const float* src = raw + row * ((size_t)H * V) + (size_t)head * V;
    float ssq = 0.f;
    for (int c = lane; c < V; c += 32) ssq += src[c] * src[c];
    ssq = warp_sum(ssq);
    const float factor = out_scale / sqrtf(ssq / (float)V + eps);
    for (int c = lane; c < V; c += 32) {
        float val = src[c] * factor;
        if (weight != nullptr) val *= weight[head * norm_head_stride + c];
        if (g != nullptr) {
            const float gate = to_float(g[row * g_stride + head * V + c]);
            val *= gate / (1.f + expf(-gate));
        }
        out[row * out_stride + head * V + c] = from_float<T>(val);
    }
}

template <typename T, int MODE, int NI, int TC, int COLS>
static int launch_scan(const ScanArgs& a, int n_seqs, cudaStream_t st) {
    const int slices = (a.V + COLS - 1) / COLS;
    if (slices > 65535) return DFI_ERR_LIMIT;
    constexpr int DP = kScanWarps * NI;
    constexpr size_t bytes = sizeof(float) * (3 * TC * DP + TC * COLS + kScanTokens * kScanWarps * COLS);
    static bool raised = false;          // per instantiation
    if (bytes > 48 * 1024 && !raised) {
        if (cudaFuncSetAttribute(linear_scan_kernel<T, MODE, NI, TC, COLS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess) {
            cudaGetLastError();
            return DFI_ERR_LAUNCH;
        }
        raised = true;
    }
    launch(linear_scan_kernel<T, MODE, NI, TC, COLS>, dim3(n_seqs, a.H, slices), dim3(kScanWarps * 32), bytes, st, a);
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

static int sm_count() {
    static int count = 0;
    if (count == 0) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0) {
            cudaGetLastError();
            count = 148;
        }
    }
    return count;
}

template <typename T, int MODE, int NI>
static int pick_fetch(const ScanArgs& a, int n_seqs, bool few_rows, cudaStream_t st) {
    // so few (sequence, head, 32 columns) that twice as many still find an SM each: 16 columns a CTA (a token
    // costs a CTA about the same either way: what it waits for is the chain through one token's sum, so a
    // second CTA on an SM would only double that SM's time; measured at 40 heads of 64 x 64, one sequence:
    // 80 CTAs of 32 columns 296 us for 2,048 tokens, 160 CTAs of 16 columns on 148 SMs 338 us)
    if constexpr (NI >= 8) {
        if (2LL * n_seqs * a.H * ((a.V + 31) / 32) <= sm_count()) {
            if (few_rows) return launch_scan<T, MODE, NI, kScanTokens, 16>(a, n_seqs, st);
            return launch_scan<T, MODE, NI, scan_fetch_tokens(NI), 16>(a, n_seqs, st);
        }
    }
    if (few_rows) return launch_scan<T, MODE, NI, kScanTokens, 32>(a, n_seqs, st);
    return launch_scan<T, MODE, NI, scan_fetch_tokens(NI), 32>(a, n_seqs, st);
}

template <typename T, int MODE>
static int pick_rows(const ScanArgs& a, int n_seqs, bool few_rows, cudaStream_t st) {
    if (a.D <= 32) return pick_fetch<T, MODE, 4>(a, n_seqs, few_rows, st);
    if (a.D <= 64) return pick_fetch<T, MODE, 8>(a, n_seqs, few_rows, st);
    if (a.D <= 128) return pick_fetch<T, MODE, 16>(a, n_seqs, few_rows, st);
    if (a.D <= 256) return pick_fetch<T, MODE, 32>(a, n_seqs, few_rows, st);
    return DFI_ERR_LIMIT;
}

// out[s][row][c] = h[row][c] + (before[c] - h[row][c]) * mu[s][c] for s < n_mix, where `before` is the
// row above in the same sequence or, for a sequence's first row of this step, the row its state holds
// (zeros when the sequence starts).  float32 arithmetic, one rounding on store.
template <typename T>
__global__ void token_shift_kernel(const T* __restrict__ h, const float* __restrict__ mu, int n_mix, int width,
                                   int rows, const float* __restrict__ state, long long slot_stride,
                                   long long carry_offset, const int* __restrict__ row_seq,
                                   const int* __restrict__ cu_rows, const int* __restrict__ seq_slot,
                                   T* __restrict__ out) {
    pdl_launch_next();
    pdl_wait();
    const int row = blockIdx.x;
    const int seq = row_seq[row];
    const bool first = row == cu_rows[seq];
    const float* kept = state + (size_t)seq_slot[seq] * slot_stride + carry_offset;
    const T* here = h + (size_t)row * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float x = to_float(here[c]);
        const float before = first ? kept[c] : to_float(here[c - width]);
        const float d = before - x;
        for (int s = 0; s < n_mix; ++s)
            out[((size_t)s * rows + row) * width + c] = from_float<T>(fmaf(d, mu[(size_t)s * width + c], x));
    }
}

}  // namespace dfi

using namespace dfi;

// mode 0: decay-then-read with a = sigmoid(z)^(1/decay_param); mode 1: read-then-decay with the bonus and
// a = exp(-exp(z)).  dtype is the storage type of q, k, v, g, out and carry_rows.  max_rows_per_seq: the most
// rows any sequence brings (0: unknown); it only picks how many tokens a fetch covers.
DFI_EXPORT int dfi_linear_scan(int mode, const void* q, int q_stride, const void* k, int k_stride, const void* v,
                               int v_stride, const void* g, int g_stride, const float* decay_logit,
                               const float* decay_bias, const float* bonus, float decay_param, float q_scale,
                               float* state, long long slot_stride, const int* cu_rows, const int* seq_slot,
                               int n_seqs, int rows, int max_rows_per_seq, int H, int D, int V, const float* norm_weight,
                               int norm_head_stride, float eps, float* raw, void* out, int out_stride,
                               float out_scale, const void* carry_rows, int carry_width, long long carry_offset,
                               int dtype, void* stream) {
    if (n_seqs <= 0) return DFI_OK;
    if (H <= 0 || H > 65535 || D <= 0 || V <= 0 || state == nullptr || decay_logit == nullptr || raw == nullptr) return DFI_ERR_SHAPE;
    if (rows <= 0) return DFI_OK;
    if (dtype != DFI_DTYPE_F32 && dtype != DFI_DTYPE_BF16) return DFI_ERR_DTYPE;
    if (mode == 1 && bonus == nullptr) return DFI_ERR_SHAPE;
    if (mode == 0 && !(decay_param > 0.f)) return DFI_ERR_SHAPE;
    ScanArgs a;
    a.q = q; a.k = k; a.v = v; a.g = g;
    a.q_stride = q_stride; a.k_stride = k_stride; a.v_stride = v_stride; a.g_stride = g_stride;
    a.decay_logit = decay_logit; a.decay_bias = decay_bias; a.bonus = bonus;
    a.decay_param = decay_param; a.q_scale = q_scale;
    a.state = state; a.slot_stride = slot_stride; a.cu_rows = cu_rows; a.seq_slot = seq_slot;
    a.H = H; a.D = D; a.V = V;
    a.raw = raw;
    a.carry_rows = carry_rows; a.carry_width = carry_width; a.carry_offset = carry_offset;
    a.bf16 = dtype == DFI_DTYPE_BF16;
    cudaStream_t st = (cudaStream_t)stream;
    int rc = DFI_ERR_SHAPE;
    const bool few = max_rows_per_seq > 0 && max_rows_per_seq <= kScanTokens;
    if (mode == 0) rc = a.bf16 ? pick_rows<bf16, 0>(a, n_seqs, few, st) : pick_rows<float, 0>(a, n_seqs, few, st);
    if (mode == 1) rc = a.bf16 ? pick_rows<bf16, 1>(a, n_seqs, few, st) : pick_rows<float, 1>(a, n_seqs, few, st);
    if (rc != DFI_OK) return rc;
    const dim3 grid(rows, (H + 3) / 4);
    if (a.bf16)
        launch(head_norm_gate_kernel<bf16>, grid, dim3(128), 0, st, (const float*)raw, H, V, norm_weight, norm_head_stride,
               eps, (const bf16*)g, g_stride, out_scale, (bf16*)out, out_stride);
    else
        launch(head_norm_gate_kernel<float>, grid, dim3(128), 0, st, (const float*)raw, H, V, norm_weight, norm_head_stride,
               eps, (const float*)g, g_stride, out_scale, (float*)out, out_stride);
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

DFI_EXPORT int dfi_token_shift(const void* h, const float* mu, int n_mix, int width, int rows, const float* state,
                               long long slot_stride, long long carry_offset, const int* row_seq,
                               const int* cu_rows, const int* seq_slot, void* out, int dtype, void* stream) {
    if (rows <= 0) return DFI_OK;
    if (n_mix <= 0 || width <= 0 || state == nullptr) return DFI_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    int threads = 32;
    while (threads < 256 && threads < width) threads <<= 1;
    if (dtype == DFI_DTYPE_F32)
        launch(token_shift_kernel<float>, rows, threads, 0, st, (const float*)h, mu, n_mix, width, rows, state,
               slot_stride, carry_offset, row_seq, cu_rows, seq_slot, (float*)out);
    else if (dtype == DFI_DTYPE_BF16)
        launch(token_shift_kernel<bf16>, rows, threads, 0, st, (const bf16*)h, mu, n_mix, width, rows, state,
               slot_stride, carry_offset, row_seq, cu_rows, seq_slot, (bf16*)out);
    else return DFI_ERR_DTYPE;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}
