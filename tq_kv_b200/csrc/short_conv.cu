// Short causal convolutions over time, one filter per channel, in front of a recurrence:
//
//   y[t, c] = act(bias[c] + sum_{j < K} w[c, K-1-j] * x[t-j, c])        (zeros before a sequence's start)
//
// x are float32 columns of a projection's result, K the number of taps (the last column of w is the current
// token's).  The K-1 inputs before a step's first token come from the sequence's state, [K-1, C] float32 per slot
// (oldest first), which a fresh slot holds as zeros; after the step it holds the sequence's last K-1 inputs.  A
// prompt, a portion of a prompt and a decoded token are therefore the same kernel.
//
// What follows the convolution in such mixers rides along:
//   * the channels are cut into regions of vectors (a head's query, key or value); a region may ask for each of
//     its vectors to be scaled to unit length, x * scale / sqrt(sum(x^2) + eps);
//   * the per-token scalars of a recurrence with one decay per head:  with sp = softplus(raw[t, h] + dt_bias[h]),
//     g = exp(-exp(A_log[h]) * sp), and second = sigmoid(beta_raw[t, h]) if given, else sp.  They are written as
//     [T, H, 4] floats (g, second, 0, 0), the layout the scan kernels stage with 16-byte copies.
//
// A warp owns one (token, vector); a lane holds up to CONV_MAX_PER_LANE of its channels.  Steps in which every
// sequence brings one token shift the state in the same kernel; otherwise a second, small kernel (a thread per
// sequence and channel, which first gathers its K-1 values and then writes them) does it after the first.
#include "common.cuh"

#define CONV_MAX_TAPS 16
#define CONV_MAX_PER_LANE 8          // vectors of up to 256 channels
#define CONV_MAX_REGIONS 4

struct ConvRegion {
    int first, count, width;         // channels first .. first + count - 1 in vectors of `width`
    int unit;                        // scale every vector to unit length
    float scale;                     // ... times this
    int vec0;                        // index of the region's first vector among all vectors
};

struct ConvArgs {
    const float* x; int ldx;
    const float* w; const float* bias;
    float* out; int ldo;
    float* state; size_t state_stride;
    const int* tok_seq; const int* cu_seqlens; const int* slots;
    int C, K, T, silu, single, n_vec, n_reg;
    ConvRegion reg[CONV_MAX_REGIONS];
    float unit_eps;
    // scalars of the recurrence (H == 0: none)
    const float* gate_raw; int ldg;
    const float* beta_raw; int ldb;
    const float* A_log; const float* dt_bias;
    float* scal; int H;
};

__device__ __forceinline__ float conv_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

template <bool SINGLE>
__global__ void __launch_bounds__(128) short_conv_kernel(ConvArgs a) {
    const int warp_global = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    pdl_wait();
    pdl_launch();
    const int n_rows = a.T * a.n_vec;
    if (warp_global >= n_rows) {
        // the warps past the vectors make the scalars: a thread per (token, head)
        const long long idx = (long long)(warp_global - n_rows) * 32 + lane;
        if (a.H > 0 && idx < (long long)a.T * a.H) {
            const int t = (int)(idx / a.H), h = (int)(idx - (long long)t * a.H);
            const float sp = conv_softplus(a.gate_raw[(size_t)t * a.ldg + h] + a.dt_bias[h]);
            const float g = expf(-expf(a.A_log[h]) * sp);
            const float second = a.beta_raw ? 1.f / (1.f + expf(-a.beta_raw[(size_t)t * a.ldb + h])) : sp;
            *reinterpret_cast<float4*>(a.scal + (size_t)idx * 4) = make_float4(g, second, 0.f, 0.f);
        }
        return;
    }
    const int t = warp_global / a.n_vec, v = warp_global - t * a.n_vec;
    int r = 0;
#pragma unroll
    for (int i = 1; i < CONV_MAX_REGIONS; ++i)
        if (i < a.n_reg && v >= a.reg[i].vec0) r = i;
    const ConvRegion rg = a.reg[r];
    const int c0 = rg.first + (v - rg.vec0) * rg.width;
    const int width = min(rg.width, rg.first + rg.count - c0);
    const int b = a.tok_seq[t];
    const int t0 = a.cu_seqlens[b];
    const int i_t = t - t0;                                  // the token's place among this step's tokens of b
    const int K = a.K, C = a.C;
    float* st = a.state + (size_t)a.slots[b] * a.state_stride;      // [K-1, C]
    float vals[CONV_MAX_PER_LANE];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < CONV_MAX_PER_LANE; ++u) {
        const int i = lane + 32 * u;
        vals[u] = 0.f;
        if (i < width) {
            const int c = c0 + i;
            // four taps at a time: first their loads (which do not wait for one another), then the sums and,
            // in a one-token step, the state's new rows (row j - 1 takes what row j held)
            float acc = a.bias ? a.bias[c] : 0.f;
            for (int j0 = 0; j0 < K; j0 += 4) {
                float xin[4];
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const int j = j0 + jj;
                    const int idx = i_t - (K - 1) + j;       // input idx of this step (negative: from the state)
                    xin[jj] = 0.f;
                    if (j < K) xin[jj] = idx >= 0 ? a.x[(size_t)(t0 + idx) * a.ldx + c] : st[(size_t)(K - 1 + idx) * C + c];
                }
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const int j = j0 + jj;
                    if (j < K) {
                        acc = fmaf(a.w[(size_t)c * K + j], xin[jj], acc);
                        if (SINGLE && j > 0) st[(size_t)(j - 1) * C + c] = xin[jj];
                    }
                }
            }
            if (a.silu) acc = acc / (1.f + expf(-acc));
            vals[u] = acc;
            ss = fmaf(acc, acc, ss);
        }
    }
    float mul = 1.f;
    if (rg.unit) {
        ss = warp_sum(ss);
        mul = rg.scale / sqrtf(ss + a.unit_eps);
    }
#pragma unroll
    for (int u = 0; u < CONV_MAX_PER_LANE; ++u) {
        const int i = lane + 32 * u;
        if (i < width) a.out[(size_t)t * a.ldo + c0 + i] = vals[u] * mul;
    }
}

// After a step of several tokens: the state of sequence b becomes the last K-1 inputs (of this step, and of the old
// state where the step brought fewer).
__global__ void short_conv_state_kernel(ConvArgs a, int n_seqs) {
    pdl_wait();
    pdl_launch();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_seqs * a.C) return;
    const int b = (int)(idx / a.C), c = (int)(idx - (long long)b * a.C);
    const int t0 = a.cu_seqlens[b], n = a.cu_seqlens[b + 1] - t0;
    const int K = a.K, C = a.C;
    if (n <= 0) return;
    float* st = a.state + (size_t)a.slots[b] * a.state_stride;
    float keep[CONV_MAX_TAPS - 1];
#pragma unroll
    for (int r = 0; r < CONV_MAX_TAPS - 1; ++r) {
        if (r < K - 1) {
            const int i = n - (K - 1) + r;
            keep[r] = i >= 0 ? a.x[(size_t)(t0 + i) * a.ldx + c] : st[(size_t)(K - 1 + i) * C + c];
        }
    }
#pragma unroll
    for (int r = 0; r < CONV_MAX_TAPS - 1; ++r)
        if (r < K - 1) st[(size_t)r * C + c] = keep[r];
}

// regions: n_reg rows of (first, count, width, unit) ints and the scales as floats.  gate_raw == null: no scalars.
TQ_API int tq_short_conv(const float* x, int ldx, const float* w, const float* bias, float* out, int ldo, float* state,
                         long long state_stride, const int* tok_seq, const int* cu_seqlens, const int* slots,
                         int n_seqs, int n_tokens, int C, int K, int silu, int single, int n_reg, const int* regions,
                         const float* scales, float unit_eps, const float* gate_raw, int ldg, const float* beta_raw,
                         int ldb, const float* A_log, const float* dt_bias, float* scal, int H, cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (!x || !w || !out || (!state && K > 1) || !tok_seq || !cu_seqlens || !slots || C <= 0 || K < 1 || K > CONV_MAX_TAPS ||
        n_reg < 1 || n_reg > CONV_MAX_REGIONS || !regions || !scales || state_stride < (long long)(K - 1) * C)
        return (int)cudaErrorInvalidValue;
    if (single && n_tokens != n_seqs) return (int)cudaErrorInvalidValue;
    ConvArgs a{};
    a.x = x; a.ldx = ldx; a.w = w; a.bias = bias; a.out = out; a.ldo = ldo; a.state = state;
    a.state_stride = (size_t)state_stride; a.tok_seq = tok_seq; a.cu_seqlens = cu_seqlens; a.slots = slots;
    a.C = C; a.K = K; a.T = n_tokens; a.silu = silu; a.single = single; a.n_reg = n_reg; a.unit_eps = unit_eps;
    int n_vec = 0;
    for (int i = 0; i < n_reg; ++i) {
        ConvRegion& r = a.reg[i];
        r.first = regions[4 * i]; r.count = regions[4 * i + 1]; r.width = regions[4 * i + 2]; r.unit = regions[4 * i + 3];
        r.scale = scales[i];
        if (r.first < 0 || r.count <= 0 || r.width <= 0 || r.width > 32 * CONV_MAX_PER_LANE || r.first + r.count > C ||
            (r.unit && r.count % r.width))
            return (int)cudaErrorInvalidValue;
        r.vec0 = n_vec;
        n_vec += (r.count + r.width - 1) / r.width;
    }
    a.n_vec = n_vec;
    long long warps = (long long)n_tokens * n_vec;
    if (gate_raw) {
        if (!A_log || !dt_bias || !scal || H <= 0) return (int)cudaErrorInvalidValue;
        a.gate_raw = gate_raw; a.ldg = ldg; a.beta_raw = beta_raw; a.ldb = ldb; a.A_log = A_log; a.dt_bias = dt_bias;
        a.scal = scal; a.H = H;
        warps += ((long long)n_tokens * H + 31) / 32;
    }
    const long long blocks = (warps + 3) / 4;
    if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
    int st = single ? tq_launch_pdl(TQ_PDL_ELEMENTWISE, short_conv_kernel<true>, dim3((unsigned)blocks), dim3(128), 0, stream, a)
                    : tq_launch_pdl(TQ_PDL_ELEMENTWISE, short_conv_kernel<false>, dim3((unsigned)blocks), dim3(128), 0, stream, a);
    if (st || single || K == 1) return st;
    const long long n = (long long)n_seqs * C;
    return tq_launch_pdl(TQ_PDL_ELEMENTWISE, short_conv_state_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0,
                         stream, a, n_seqs);
}
