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
// One CTA of eight warps owns one (sequence, head) for all the tokens the step brings it.  Warp w keeps
// rows [w NI, (w+1) NI) of S in registers, lane c the columns c, c + 32, ...; tokens are taken sixteen at
// a time: their q, k, decays and v are staged in shared memory as float32 (the decay computed once per
// token and channel), every warp leaves its share of o_t there, and after the sixteen tokens the warps
// sum the shares token by token, divide a head's output by its root mean square, weight it, gate it with
// silu(g) and store it: the norm and the gate cost no pass of their own.
//
// The token shift of the time-mixing layer (every projection reads its own blend of a token's row and
// the row before it) is the other kernel here; the row that a sequence's next step will need lives in
// the same state area as S and is written by the scan kernel, which runs after the blends were read.
#include "common.cuh"

namespace dfi {

constexpr int kScanWarps = 8;
constexpr int kScanTokens = 16;

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
    const float* norm_weight;      // [V] (norm_head_stride 0) or [H, V] (norm_head_stride V); null: no weight
    int norm_head_stride;
    float eps;
    void* out; int out_stride;     // [rows, out_stride]: H heads of V
    float out_scale;
    const void* carry_rows;        // or null: [rows, carry_width] rows whose last one per sequence is kept in the state
    int carry_width;
    long long carry_offset;        // where in a slot that row lives
    int bf16;                      // storage type of q, k, v, g, out, carry_rows
};

__device__ __forceinline__ float load_as_float(const void* p, size_t i, int is_bf16) {
    return is_bf16 ? __bfloat162float(reinterpret_cast<const bf16*>(p)[i]) : reinterpret_cast<const float*>(p)[i];
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

template <int MODE, int NI, int NC>
__global__ void __launch_bounds__(kScanWarps * 32) linear_scan_kernel(const ScanArgs a) {
    extern __shared__ __align__(16) float smem[];
    constexpr int DP = kScanWarps * NI, VP = 32 * NC, TC = kScanTokens;
    float* rs = smem;                    // [TC][DP]
    float* ks = rs + TC * DP;            // [TC][DP]
    float* ws = ks + TC * DP;            // [TC][DP]
    float* vs = ws + TC * DP;            // [TC][VP]
    float* op = vs + TC * VP;            // [TC][warps][VP]
    pdl_launch_next();
    pdl_wait();
    const int seq = blockIdx.x, head = blockIdx.y;
    const int row0 = a.cu_rows[seq], row1 = a.cu_rows[seq + 1];
    if (row1 <= row0) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int D = a.D, V = a.V, HD = a.H * a.D;
    float* S_g = a.state + (size_t)a.seq_slot[seq] * a.slot_stride + (size_t)head * D * V;
    const int i0 = warp * NI;

    float S[NC][NI], U[NI];
#pragma unroll
    for (int n = 0; n < NI; ++n) {
        const int i = i0 + n;
        U[n] = (MODE == 1 && i < D) ? a.bonus[head * D + i] : 0.f;
#pragma unroll
        for (int m = 0; m < NC; ++m) {
            const int j = lane + 32 * m;
            S[m][n] = (i < D && j < V) ? S_g[(size_t)i * V + j] : 0.f;
        }
    }

    for (int c0 = row0; c0 < row1; c0 += TC) {
        const int nt = min(TC, row1 - c0);
        __syncthreads();
        for (int idx = tid; idx < nt * DP; idx += kScanWarps * 32) {
            const int t = idx / DP, i = idx - t * DP;
            const size_t row = (size_t)(c0 + t);
            float r = 0.f, k = 0.f, w = 1.f;
            if (i < D) {
                const int col = head * D + i;
                r = load_as_float(a.q, row * a.q_stride + col, a.bf16) * a.q_scale;
                k = load_as_float(a.k, row * a.k_stride + col, a.bf16);
                float z = a.decay_logit[row * HD + col];
                if (a.decay_bias != nullptr) z += a.decay_bias[col];
                w = decay_of<MODE>(z, a.decay_param);
            }
            rs[idx] = r; ks[idx] = k; ws[idx] = w;
        }
        for (int idx = tid; idx < nt * VP; idx += kScanWarps * 32) {
            const int t = idx / VP, j = idx - t * VP;
            vs[idx] = j < V ? load_as_float(a.v, (size_t)(c0 + t) * a.v_stride + head * V + j, a.bf16) : 0.f;
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            float o[NC], vj[NC];
#pragma unroll
            for (int m = 0; m < NC; ++m) { o[m] = 0.f; vj[m] = vs[t * VP + lane + 32 * m]; }
            const float4* r4 = reinterpret_cast<const float4*>(rs + t * DP + i0);
            const float4* k4 = reinterpret_cast<const float4*>(ks + t * DP + i0);
            const float4* w4 = reinterpret_cast<const float4*>(ws + t * DP + i0);
#pragma unroll
            for (int n4 = 0; n4 < NI / 4; ++n4) {
                const float4 rv = r4[n4], kv4 = k4[n4], wv = w4[n4];
                const float r[4] = {rv.x, rv.y, rv.z, rv.w}, k[4] = {kv4.x, kv4.y, kv4.z, kv4.w}, w[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int n = n4 * 4 + e;
#pragma unroll
                    for (int m = 0; m < NC; ++m) {
                        if (MODE == 0) {
                            S[m][n] = fmaf(w[e], S[m][n], k[e] * vj[m]);
                            o[m] = fmaf(r[e], S[m][n], o[m]);
                        } else {
                            const float kv = k[e] * vj[m];
                            o[m] = fmaf(r[e], fmaf(U[n], kv, S[m][n]), o[m]);
                            S[m][n] = fmaf(w[e], S[m][n], kv);
                        }
                    }
                }
            }
#pragma unroll
            for (int m = 0; m < NC; ++m) op[(t * kScanWarps + warp) * VP + lane + 32 * m] = o[m];
        }
        __syncthreads();
        // the sixteen tokens' outputs: sum the warps' shares, unit root mean square over V, weight, gate
        for (int t = warp; t < nt; t += kScanWarps) {
            const size_t row = (size_t)(c0 + t);
            float o[NC], ssq = 0.f;
#pragma unroll
            for (int m = 0; m < NC; ++m) {
                float sum = 0.f;
#pragma unroll
                for (int w8 = 0; w8 < kScanWarps; ++w8) sum += op[(t * kScanWarps + w8) * VP + lane + 32 * m];
                o[m] = sum;
                ssq += sum * sum;           // columns from V on are zero
            }
            ssq = warp_sum(ssq);
            const float factor = a.out_scale / sqrtf(ssq / (float)V + a.eps);
#pragma unroll
            for (int m = 0; m < NC; ++m) {
                const int j = lane + 32 * m;
                if (j < V) {
                    float val = o[m] * factor;
                    if (a.norm_weight != nullptr) val *= a.norm_weight[head * a.norm_head_stride + j];
                    if (a.g != nullptr) {
                        const float gate = load_as_float(a.g, row * a.g_stride + head * V + j, a.bf16);
                        val *= gate / (1.f + expf(-gate));
                    }
                    store_from_float(a.out, row * a.out_stride + head * V + j, val, a.bf16);
                }
            }
        }
    }
#pragma unroll
    for (int n = 0; n < NI; ++n) {
        const int i = i0 + n;
#pragma unroll
        for (int m = 0; m < NC; ++m) {
            const int j = lane + 32 * m;
            if (i < D && j < V) S_g[(size_t)i * V + j] = S[m][n];
        }
    }
    if (a.carry_rows != nullptr && head == 0) {
        float* dst = a.state + (size_t)a.seq_slot[seq] * a.slot_stride + a.carry_offset;
        for (int c = tid; c < a.carry_width; c += kScanWarps * 32)
            dst[c] = load_as_float(a.carry_rows, (size_t)(row1 - 1) * a.carry_width + c, a.bf16);
    }
}

template <int MODE, int NI, int NC>
static int launch_scan(const ScanArgs& a, int n_seqs, cudaStream_t st) {
    constexpr int DP = kScanWarps * NI, VP = 32 * NC;
    const size_t bytes = sizeof(float) * kScanTokens * (3 * DP + VP + kScanWarps * VP);
    if (bytes > 48 * 1024) {
        static bool raised = false;          // per instantiation
        if (!raised) {
            if (cudaFuncSetAttribute(linear_scan_kernel<MODE, NI, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)bytes) != cudaSuccess) {
                cudaGetLastError();
                return DFI_ERR_LAUNCH;
            }
            raised = true;
        }
    }
    launch(linear_scan_kernel<MODE, NI, NC>, dim3(n_seqs, a.H), dim3(kScanWarps * 32), bytes, st, a);
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

template <int MODE, int NI>
static int pick_columns(const ScanArgs& a, int n_seqs, cudaStream_t st) {
    if (a.V <= 32) return launch_scan<MODE, NI, 1>(a, n_seqs, st);
    if (a.V <= 64) return launch_scan<MODE, NI, 2>(a, n_seqs, st);
    if (a.V <= 128) return launch_scan<MODE, NI, 4>(a, n_seqs, st);
    if constexpr (NI <= 16) {
        if (a.V <= 256) return launch_scan<MODE, NI, 8>(a, n_seqs, st);
    }
    return DFI_ERR_LIMIT;
}

template <int MODE>
static int pick_rows(const ScanArgs& a, int n_seqs, cudaStream_t st) {
    if (a.D <= 32) return pick_columns<MODE, 4>(a, n_seqs, st);
    if (a.D <= 64) return pick_columns<MODE, 8>(a, n_seqs, st);
    if (a.D <= 128) return pick_columns<MODE, 16>(a, n_seqs, st);
    if (a.D <= 256) return pick_columns<MODE, 32>(a, n_seqs, st);
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
// a = exp(-exp(z)).  dtype is the storage type of q, k, v, g, out and carry_rows.
DFI_EXPORT int dfi_linear_scan(int mode, const void* q, int q_stride, const void* k, int k_stride, const void* v,
                               int v_stride, const void* g, int g_stride, const float* decay_logit,
                               const float* decay_bias, const float* bonus, float decay_param, float q_scale,
                               float* state, long long slot_stride, const int* cu_rows, const int* seq_slot,
                               int n_seqs, int H, int D, int V, const float* norm_weight, int norm_head_stride,
                               float eps, void* out, int out_stride, float out_scale, const void* carry_rows,
                               int carry_width, long long carry_offset, int dtype, void* stream) {
    if (n_seqs <= 0) return DFI_OK;
    if (H <= 0 || H > 65535 || D <= 0 || V <= 0 || state == nullptr || decay_logit == nullptr) return DFI_ERR_SHAPE;
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
    a.norm_weight = norm_weight; a.norm_head_stride = norm_head_stride; a.eps = eps;
    a.out = out; a.out_stride = out_stride; a.out_scale = out_scale;
    a.carry_rows = carry_rows; a.carry_width = carry_width; a.carry_offset = carry_offset;
    a.bf16 = dtype == DFI_DTYPE_BF16;
    cudaStream_t st = (cudaStream_t)stream;
    if (mode == 0) return pick_rows<0>(a, n_seqs, st);
    if (mode == 1) return pick_rows<1>(a, n_seqs, st);
    return DFI_ERR_SHAPE;
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
