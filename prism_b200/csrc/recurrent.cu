// Recurrent mixers: layers whose memory of a sequence is a matrix of fixed size per head instead of a cache of
// keys.  Two recurrences share one scan kernel; S is [dk, dv] per head, float32, one per request slot:
//
//   delta rule with a scalar decay (SCAN_DELTA), per token with unit-length q, k and g, beta in (0, 1):
//       S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (the read-out sees this token's write)
//   decayed outer-product sum with a bonus for the current token (SCAN_BONUS), w, u vectors over the key channels:
//       o = (S + diag(u) k v^T)^T r;   S <- diag(w) S + k v^T                    (the read-out sees S before the write)
//
// Everything that enters the recurrence is float32: the kernels here read the float32 results of the input
// projections, and the state never leaves float32.  A request's state lives in its slot between steps, so
// the result at a position does not depend on how the request was cut into steps: the scan visits the
// tokens one after another either way, and the order of additions inside a token depends on the sizes only.
//
// Around the scans:
//   * prism_conv_unit_gates  per token: the short causal convolution over time of the q | k | v channels (its
//     last taps - 1 inputs per request are state too) with silu, q and k made unit vectors per head (q also
//     times dk^-1/2), beta = sigmoid(b), g = exp(-exp(A_log) softplus(a + dt_bias));
//   * prism_state_tail       the last rows of a step's input per request into a [slots, rows, width] state (the
//     convolution's tail; with one row, the previous token's input of a token-shift mix);
//   * prism_shift_mix        x + (x_prev - x) mu_s for several mu at once (x_prev of a step's first token comes
//     from the state);
//   * prism_headnorm_gate    o / rms(o) per head, times a weight, times silu(gate), times a constant.
#include "common.cuh"

#define PRISM_SCAN_DELTA 0
#define PRISM_SCAN_BONUS 1

namespace prism {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ---------------------------------------------------------------------------------------------------------
// conv + silu, unit vectors, gates.  One CTA per token.
//   proj   [T, *] float32, row stride ps: columns [0, C) are the q | k | v channels (C = 2 G dk + H dv),
//          columns ob .. ob + H the beta projection, oa .. oa + H the decay projection
//   taps   [C, K] (last column: the current token's)
//   tail   [slots, K - 1, C] float32: the K - 1 inputs before the step's first token, oldest first
//   qkv    [T, C] float32 out;   bg [T, 2 H] float32 out: beta | g
// ---------------------------------------------------------------------------------------------------------
__global__ void conv_unit_gates_kernel(const float* __restrict__ proj_in, long long ps, int ob, int oa,
                                       const void* __restrict__ taps, int taps_bf16, int K,
                                       const float* __restrict__ tail, const void* __restrict__ a_log, int a_log_bf16,
                                       const void* __restrict__ dt_bias, int dt_bf16, const int* __restrict__ tok_seg,
                                       const int* __restrict__ seg_start, const int* __restrict__ slots, int G, int H,
                                       int dk, int dv, float unit_eps, float* __restrict__ qkv, float* __restrict__ bg) {
    pdl_trigger();
    pdl_wait();
    const float* proj = pdl_fresh(proj_in);
    extern __shared__ float y[];                       // [C]
    const int t = blockIdx.x, seg = tok_seg[t];
    const int i = t - seg_start[seg];                  // place of the token in its segment
    const int C = 2 * G * dk + H * dv;
    const float* tl = tail + (size_t)slots[seg] * (K - 1) * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = 0.f;
        for (int j = K - 1; j >= 0; --j) {             // lag j: the input j tokens back; oldest first
            const int src = i - j;
            const float x = src >= 0 ? proj[(size_t)(t - j) * ps + c] : tl[(size_t)(K - 1 + src) * C + c];
            acc += load_param(taps, taps_bf16, (size_t)c * K + (K - 1 - j)) * x;
        }
        y[c] = silu_f(acc);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    float* out = qkv + (size_t)t * C;
    for (int hh = warp; hh < 2 * G; hh += nwarps) {    // q heads, then k heads
        const float* row = y + hh * dk;
        float ss = 0.f;
        for (int d = lane; d < dk; d += 32) ss += row[d] * row[d];
        ss = warp_sum(ss);
        const float inv = (1.f / sqrtf(ss + unit_eps)) * (hh < G ? 1.f / sqrtf((float)dk) : 1.f);
        for (int d = lane; d < dk; d += 32) out[hh * dk + d] = row[d] * inv;
    }
    for (int c = 2 * G * dk + threadIdx.x; c < C; c += blockDim.x) out[c] = y[c];
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        bg[(size_t)t * 2 * H + h] = sigmoid_f(proj[(size_t)t * ps + ob + h]);
        const float dt = softplus_f(proj[(size_t)t * ps + oa + h] + load_param(dt_bias, dt_bf16, h));
        bg[(size_t)t * 2 * H + H + h] = expf(-expf(load_param(a_log, a_log_bf16, h)) * dt);
    }
}

// tail[slot][r][c] <- the input (rows - r) tokens before the end of the request's tokens so far: from this
// step's rows where the step reaches that far back, else from the tail as it was (shifted).  One CTA per
// segment; a thread owns a column, and walks r upwards, so that what it still needs is never overwritten.
__global__ void state_tail_kernel(const float* __restrict__ src_in, long long ss, int width, float* __restrict__ tail,
                                  int rows, const int* __restrict__ seg_start, const int* __restrict__ slots) {
    pdl_trigger();
    pdl_wait();
    const float* src = pdl_fresh(src_in);
    const int seg = blockIdx.x, s0 = seg_start[seg], qlen = seg_start[seg + 1] - s0;
    float* tl = tail + (size_t)slots[seg] * rows * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x)
        for (int r = 0; r < rows; ++r) {
            const int idx = qlen - rows + r;           // place in the segment of the token that row r holds afterwards
            tl[(size_t)r * width + c] = idx >= 0 ? src[(size_t)(s0 + idx) * ss + c] : tl[(size_t)(r + qlen) * width + c];
        }
}

// out[s][t][c] = x[t][c] + (x_prev[t][c] - x[t][c]) mu[s][c],  s < n;  x_prev of a segment's first token is prev[slot].
template <typename T>
__global__ void shift_mix_kernel(const float* __restrict__ x_in, int D, const float* __restrict__ prev,
                                 const void* __restrict__ mu, int mu_bf16, int n, const int* __restrict__ tok_seg,
                                 const int* __restrict__ seg_start, const int* __restrict__ slots, T* __restrict__ out,
                                 long long out_plane) {
    pdl_trigger();
    pdl_wait();
    const float* x = pdl_fresh(x_in);
    const int t = blockIdx.x, seg = tok_seg[t];
    const float* xp = t > seg_start[seg] ? x + (size_t)(t - 1) * D : prev + (size_t)slots[seg] * D;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        const float a = x[(size_t)t * D + c], d = xp[c] - a;
        for (int s = 0; s < n; ++s)
            out[(size_t)s * out_plane + (size_t)t * D + c] = from_float<T>(a + d * load_param(mu, mu_bf16, (size_t)s * D + c));
    }
}

// out[t][h dv + c] = o[t][h][c] / sqrt(mean_c(o[t][h]^2) + eps) * weight[widx] * silu(gate[t][h dv + c]) * scale,
// widx = c (one weight for all heads) or h dv + c (per_head_weight).  One warp per (token, head).
template <typename T>
__global__ void headnorm_gate_kernel(const float* __restrict__ o_in, const float* __restrict__ gate_in, long long gs,
                                     const void* __restrict__ weight, int weight_bf16, int per_head_weight, float eps,
                                     float scale, int Ttot, int H, int dv, T* __restrict__ out, long long os) {
    pdl_trigger();
    pdl_wait();
    const float* o = pdl_fresh(o_in);
    const float* gate = pdl_fresh(gate_in);
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= (long long)Ttot * H) return;
    const int t = (int)(w / H), h = (int)(w % H);
    const float* row = o + ((size_t)t * H + h) * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss += row[c] * row[c];
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)dv + eps);
    for (int c = lane; c < dv; c += 32) {
        const float wv = load_param(weight, weight_bf16, per_head_weight ? (size_t)h * dv + c : (size_t)c);
        const float g = silu_f(gate[(size_t)t * gs + (size_t)h * dv + c]);
        out[(size_t)t * os + (size_t)h * dv + c] = from_float<T>(row[c] * inv * wv * g * scale);
    }
}

// ---------------------------------------------------------------------------------------------------------
// The scan.  grid (heads, segments, column blocks); a thread owns R rows (i = part + L n) of one column of S,
// the L threads of a column are neighbouring lanes of a warp and add up their partial dot products by shuffles.
// The step's vectors come through shared memory TB tokens at a time.  The state is kept in memory as
// [slot][head][column][row], so that the L threads of a column read neighbouring floats.
//   SCAN_DELTA:  qk [T, *] row stride qs: q of kv head g at qo + g dk, k at ko + g dk; v at vo + h dv;
//                bg [T, 2 H]: beta | g.
//   SCAN_BONUS:  r at qo + h dk, k at ko + h dk, v at vo + h dv (dk == dv there), the decay's exponent ww
//                [T, H dk] (row stride ws) with w = exp(-exp(ww + w0)), w0 [H dk], bonus u [H dk].
// ---------------------------------------------------------------------------------------------------------
struct ScanArgs {
    const float* x;          // q | k | v (or r | k | v) rows
    long long xs;
    int qo, ko, vo;
    const float* bg;         // DELTA: beta | g
    const float* ww;         // BONUS: the decay's exponent before w0
    long long ws;
    const void* w0;
    int w0_bf16;
    const void* u;
    int u_bf16;
    float* state;            // [slots, H, dv, dk]
    const int* seg_start;
    const int* slots;
    float* out;              // [T, H, dv]
    int H, rep, dk, dv, cols, L, TB;
};

template <int MODE, int R>
__global__ void scan_kernel(const ScanArgs a) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float sm[];
    const int h = blockIdx.x, seg = blockIdx.y, col0 = blockIdx.z * a.cols;
    const int s0 = a.seg_start[seg], qlen = a.seg_start[seg + 1] - s0;
    const int L = a.L, dk = a.dk, dv = a.dv, TB = a.TB;
    const int ncols = min(a.cols, dv - col0);
    // the block is a whole number of warps: threads beyond the CTA's columns run along (they take part in the
    // shuffles) and neither load nor store
    const int part = threadIdx.x % L;
    const bool live = (int)threadIdx.x / L < ncols;
    const int lc = live ? threadIdx.x / L : 0, col = col0 + lc;
    const int kvh = h / a.rep;                         // DELTA: the q/k head this head uses
    // shared: per token of the block  first[dk] (q or r) | second[dk] (k) | third[dk] (BONUS: w) | v[cols] | 2 scalars
    const int per_tok = (MODE == PRISM_SCAN_BONUS ? 3 : 2) * dk + a.cols + 2;
    float* ub = sm + (size_t)TB * per_tok;             // BONUS: u[dk]
    float S[R];
    float* st = a.state + (((size_t)a.slots[seg] * a.H + h) * dv + (live ? col : 0)) * dk;
#pragma unroll
    for (int n = 0; n < R; ++n) {
        const int i = part + L * n;
        S[n] = (live && i < dk) ? st[i] : 0.f;
    }
    if (MODE == PRISM_SCAN_BONUS)
        for (int i = threadIdx.x; i < dk; i += blockDim.x) ub[i] = load_param(a.u, a.u_bf16, (size_t)h * dk + i);
    const float* x = pdl_fresh(a.x);
    const float* bg = pdl_fresh(a.bg);
    const float* ww = pdl_fresh(a.ww);

    for (int b0 = 0; b0 < qlen; b0 += TB) {
        const int nb = min(TB, qlen - b0);
        __syncthreads();                               // the block before this one has been used up
        for (int idx = threadIdx.x; idx < nb * per_tok; idx += blockDim.x) {
            const int tt = idx / per_tok, c = idx - tt * per_tok;
            const size_t t = (size_t)(s0 + b0 + tt);
            float v;
            if (MODE == PRISM_SCAN_DELTA) {
                if (c < dk) v = x[t * a.xs + a.qo + kvh * dk + c];
                else if (c < 2 * dk) v = x[t * a.xs + a.ko + kvh * dk + (c - dk)];
                else if (c < 2 * dk + a.cols) v = (c - 2 * dk) < ncols ? x[t * a.xs + a.vo + h * dv + col0 + (c - 2 * dk)] : 0.f;
                else v = bg[t * 2 * a.H + (c - 2 * dk - a.cols) * a.H + h];          // beta, then g
            } else {
                if (c < dk) v = x[t * a.xs + a.qo + h * dk + c];
                else if (c < 2 * dk) v = x[t * a.xs + a.ko + h * dk + (c - dk)];
                else if (c < 3 * dk) {
                    const int i = c - 2 * dk;
                    v = expf(-expf(ww[t * a.ws + h * dk + i] + load_param(a.w0, a.w0_bf16, (size_t)h * dk + i)));
                } else if (c < 3 * dk + a.cols) v = (c - 3 * dk) < ncols ? x[t * a.xs + a.vo + h * dv + col0 + (c - 3 * dk)] : 0.f;
                else v = 0.f;
            }
            sm[idx] = v;
        }
        __syncthreads();
        for (int tt = 0; tt < nb; ++tt) {
            const float* f1 = sm + (size_t)tt * per_tok;           // q or r
            const float* f2 = f1 + dk;                             // k
            float o;
            if (MODE == PRISM_SCAN_DELTA) {
                const float* vv = f2 + dk;
                const float beta = vv[a.cols], g = vv[a.cols + 1];
                float ks = 0.f;
#pragma unroll
                for (int n = 0; n < R; ++n) {
                    const int i = part + L * n;
                    if (i < dk) ks += S[n] * f2[i];
                }
                for (int off = L >> 1; off > 0; off >>= 1) ks += __shfl_xor_sync(0xffffffffu, ks, off);
                const float uu = beta * (vv[lc] - g * ks);
                o = 0.f;
#pragma unroll
                for (int n = 0; n < R; ++n) {
                    const int i = part + L * n;
                    if (i < dk) {
                        S[n] = g * S[n] + f2[i] * uu;
                        o += S[n] * f1[i];
                    }
                }
            } else {
                const float* wd = f2 + dk;
                const float v = wd[dk + lc];
                o = 0.f;
#pragma unroll
                for (int n = 0; n < R; ++n) {
                    const int i = part + L * n;
                    if (i < dk) {
                        const float kv = f2[i] * v;
                        o += f1[i] * (S[n] + ub[i] * kv);
                        S[n] = wd[i] * S[n] + kv;
                    }
                }
            }
            for (int off = L >> 1; off > 0; off >>= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
            if (live && part == 0) a.out[((size_t)(s0 + b0 + tt) * a.H + h) * dv + col] = o;
        }
    }
    if (live) {
#pragma unroll
        for (int n = 0; n < R; ++n) {
            const int i = part + L * n;
            if (i < dk) st[i] = S[n];
        }
    }
}

template <int MODE, int R>
static int launch_scan(const ScanArgs& a, int S, cudaStream_t stream) {
    const int per_tok = (MODE == PRISM_SCAN_BONUS ? 3 : 2) * a.dk + a.cols + 2;
    const size_t smem = ((size_t)a.TB * per_tok + (MODE == PRISM_SCAN_BONUS ? a.dk : 0)) * sizeof(float);
    auto kern = scan_kernel<MODE, R>;
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    dim3 grid(a.H, S, (a.dv + a.cols - 1) / a.cols);
    return (int)launch_kernel(kern, grid, dim3((a.cols * a.L + 31) / 32 * 32), smem, stream, a);
}

}  // namespace prism

PRISM_EXPORT int prism_conv_unit_gates(const float* proj, long long ps, int ob, int oa, const void* taps, int taps_dtype,
                                       int K, const float* tail, const void* a_log, int a_log_dtype, const void* dt_bias,
                                       int dt_dtype, const int* tok_seg, const int* seg_start, const int* slots, int T, int G,
                                       int H, int dk, int dv, float unit_eps, float* qkv, float* bg, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (K < 1 || G < 1 || H < 1 || dk < 1 || dv < 1) return (int)cudaErrorInvalidValue;
    const int C = 2 * G * dk + H * dv;
    const size_t smem = (size_t)C * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    auto kern = prism::conv_unit_gates_kernel;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return (int)prism::launch_kernel(kern, dim3(T), dim3(C >= 2048 ? 256 : 128), smem, stream, proj, ps, ob, oa, taps,
                                     taps_dtype == PRISM_DTYPE_BF16, K, tail, a_log, a_log_dtype == PRISM_DTYPE_BF16, dt_bias,
                                     dt_dtype == PRISM_DTYPE_BF16, tok_seg, seg_start, slots, G, H, dk, dv, unit_eps, qkv, bg);
}

PRISM_EXPORT int prism_state_tail(const float* src, long long src_stride, int width, float* tail, int rows,
                                  const int* seg_start, const int* slots, int S, cudaStream_t stream) {
    if (S <= 0 || rows <= 0 || width <= 0) return 0;
    return (int)prism::launch_kernel(prism::state_tail_kernel, dim3(S), dim3(width >= 1024 ? 256 : 128), 0, stream, src,
                                     src_stride, width, tail, rows, seg_start, slots);
}

PRISM_EXPORT int prism_shift_mix(const float* x, int D, const float* prev, const void* mu, int mu_dtype, int n,
                                 const int* tok_seg, const int* seg_start, const int* slots, int T, void* out, int out_dtype,
                                 long long out_plane, cudaStream_t stream) {
    if (T <= 0 || n <= 0) return 0;
    const int threads = D >= 1024 ? 256 : 128;
    const int mb = mu_dtype == PRISM_DTYPE_BF16;
    if (out_dtype == PRISM_DTYPE_BF16)
        return (int)prism::launch_kernel(prism::shift_mix_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, x, D, prev, mu,
                                         mb, n, tok_seg, seg_start, slots, (__nv_bfloat16*)out, out_plane);
    return (int)prism::launch_kernel(prism::shift_mix_kernel<float>, dim3(T), dim3(threads), 0, stream, x, D, prev, mu, mb, n,
                                     tok_seg, seg_start, slots, (float*)out, out_plane);
}

PRISM_EXPORT int prism_headnorm_gate(const float* o, const float* gate, long long gate_stride, const void* weight,
                                     int weight_dtype, int per_head_weight, float eps, float scale, int T, int H, int dv,
                                     void* out, int out_dtype, long long out_stride, cudaStream_t stream) {
    if (T <= 0 || H <= 0 || dv <= 0) return 0;
    const int warps = 4;
    const long long total = (long long)T * H;
    const int blocks = (int)((total + warps - 1) / warps);
    const int wb = weight_dtype == PRISM_DTYPE_BF16;
    if (out_dtype == PRISM_DTYPE_BF16)
        return (int)prism::launch_kernel(prism::headnorm_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), 0, stream, o,
                                         gate, gate_stride, weight, wb, per_head_weight, eps, scale, T, H, dv,
                                         (__nv_bfloat16*)out, out_stride);
    return (int)prism::launch_kernel(prism::headnorm_gate_kernel<float>, dim3(blocks), dim3(warps * 32), 0, stream, o, gate,
                                     gate_stride, weight, wb, per_head_weight, eps, scale, T, H, dv, (float*)out, out_stride);
}

// mode PRISM_SCAN_*; state [slots, H, dv, dk] float32; out [T, H, dv] float32; rep: heads per q/k head (DELTA).
// Returns cudaErrorInvalidValue for dk > 1024.
PRISM_EXPORT int prism_recurrent_scan(int mode, const float* x, long long x_stride, int qo, int ko, int vo, const float* bg,
                                      const float* ww, long long ww_stride, const void* w0, int w0_dtype, const void* u,
                                      int u_dtype, float* state, const int* seg_start, const int* slots, int S, int H, int rep,
                                      int dk, int dv, float* out, cudaStream_t stream) {
    using namespace prism;
    if (S <= 0) return 0;
    if (H < 1 || rep < 1 || dk < 1 || dv < 1 || dk > 1024 || S > 65535) return (int)cudaErrorInvalidValue;
    ScanArgs a;
    a.x = x; a.xs = x_stride; a.qo = qo; a.ko = ko; a.vo = vo; a.bg = bg; a.ww = ww; a.ws = ww_stride;
    a.w0 = w0; a.w0_bf16 = w0_dtype == PRISM_DTYPE_BF16; a.u = u; a.u_bf16 = u_dtype == PRISM_DTYPE_BF16;
    a.state = state; a.seg_start = seg_start; a.slots = slots; a.out = out; a.H = H; a.rep = rep; a.dk = dk; a.dv = dv;
    const int R = dk > 512 ? 32 : 16;
    int L = 1;
    while (L * R < dk) L *= 2;                          // at most 32
    a.L = L;
    a.cols = 128 / L < dv ? 128 / L : dv;              // about 128 threads a CTA
    const int per_tok = (mode == PRISM_SCAN_BONUS ? 3 : 2) * dk + a.cols + 2;
    int tb = (32 * 1024 / 4) / per_tok;
    a.TB = tb < 1 ? 1 : (tb > 16 ? 16 : tb);
    if (mode == PRISM_SCAN_DELTA)
        return R == 16 ? launch_scan<PRISM_SCAN_DELTA, 16>(a, S, stream) : launch_scan<PRISM_SCAN_DELTA, 32>(a, S, stream);
    if (mode == PRISM_SCAN_BONUS)
        return R == 16 ? launch_scan<PRISM_SCAN_BONUS, 16>(a, S, stream) : launch_scan<PRISM_SCAN_BONUS, 32>(a, S, stream);
    return (int)cudaErrorInvalidValue;
}
