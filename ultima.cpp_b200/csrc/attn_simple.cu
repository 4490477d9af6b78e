// Attention over the paged cache, one block for each (query token, query head), any head size
// up to 256, float32 or bfloat16 storage, float32 arithmetic throughout.
//
// It restates the reference's per-token loop (src/model/qwen_block.cpp:94-135): scores
// q.k * scale over the visible positions, max-shifted softmax (src/kernels/softmax.cpp:9-29),
// weighted sum of the values; query head h reads KV head h / (nh / nkv); a token at position
// p sees positions (p - window, p] (src/model/qwen_block.cpp:742-745).  Keys are taken in
// chunks with a running maximum, so the context length is not bounded by shared memory.
// The order of every sum depends only on the key range, never on the batch.
//
// Beyond the reference: values may have a head size of their own (``hd_v``); ``block`` > 0 masks by
// blocks of positions counted from the sequence's start (p sees j <= p with j / block == p / block);
// ``gate`` (float32, one number a token and head, or ``gate_wide`` one a token and output element)
// multiplies the output by its sigmoid.  Further options, all off at zero: ``keep_first`` > 0 with a
// window: the sequence's first keep_first positions stay visible behind the window; ``slopes`` (float32,
// one a head): slope * (distance to the key) is taken off a score; ``sink``: the softmax's sum has one
// more term exp(0) that brings no value (``sink_vals``, float32, one a head: the term is exp(sink_vals[h])
// instead); ``softcap`` > 0: a scaled score s becomes softcap * tanh(s / softcap); ``dist_bias`` (float32
// [n_dist, heads]): row min(distance to the key, n_dist - 1) is added to the score behind scale and cap (a
// learned bias by distance, looked up per head); ``out_scale`` multiplies the output.  Key rows may be up
// to 1,024 wide and value rows up to 512; the values may be the leading columns of the key rows (the caller
// then hands the key cache in twice, with the keys' head size as the values' row size ``v_row``).  The
// placement kernels at the end prepare queries and fill the cache from projection rows whose q, k and
// v columns lie anywhere, for layers the fused preparation of basic.cu does not take (unequal head
// sizes, no keys and values of their own, a norm over all heads at once, values that are the keys).
#include "common.cuh"

constexpr int CHUNK = 512;

template <typename TQ, typename TC>
__global__ void __launch_bounds__(128)
attn_simple_kernel(const TQ* __restrict__ q, long long q_stride, const TC* __restrict__ kc,
                   const TC* __restrict__ vc, TQ* __restrict__ out, long long o_stride,
                   const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, PagedKV c, PagedKV cv,
                   int nh, int window, int block, const float* __restrict__ gate, long long g_stride, float scale,
                   int keep_first, const float* __restrict__ slopes, int sink, int gate_wide, float out_scale,
                   float softcap, const float* __restrict__ dist_bias, int n_dist, const float* __restrict__ sink_vals,
                   int hdv) {
    extern __shared__ float smem[];
    float* qs = smem;                    // [hd]
    float* sc = smem + c.head_dim;       // [CHUNK]
    __shared__ float red[33];
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int hd = c.head_dim;
    const int kvh = h / (nh / c.n_kv_heads);
    const int pos = tok_pos[t], seq = tok_seq[t];
    int lo = 0;
    if (window > 0 && pos + 1 > window) lo = pos + 1 - window;
    if (block > 0) lo = max(lo, pos - pos % block);
    for (int i = tid; i < hd; i += blockDim.x) qs[i] = to_f32<TQ>(q[(long long)t * q_stride + (long long)h * hd + i]);
    __syncthreads();
    // the sink is a key with score 0 and no value: the running maximum and sum start from it
    float m = sink ? (sink_vals ? sink_vals[h] : 0.f) : -INFINITY, l = sink ? 1.f : 0.f;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const float inv_cap = softcap > 0.f ? 1.0f / softcap : 0.f;
    // visible keys: the kept first positions that the window has left behind, then lo .. pos
    const int n_kept = min(max(keep_first, 0), lo);
    const int n_keys = n_kept + pos + 1 - lo;
    const float slope = slopes ? slopes[h] : 0.f;
    for (int c0 = 0; c0 < n_keys; c0 += CHUNK) {
        const int n = min(CHUNK, n_keys - c0);
        float cmax = -INFINITY;
        for (int j = tid; j < n; j += blockDim.x) {
            const int key = c0 + j < n_kept ? c0 + j : lo + (c0 + j - n_kept);
            const TC* kr = kc + paged_offset(c, seq, key, kvh);
            float s = 0.f;
            for (int i = 0; i < hd; ++i) s = fmaf(qs[i], to_f32<TC>(kr[i]), s);
            s = s * scale;
            if (softcap > 0.f) s = softcap * tanhf(s * inv_cap);
            s -= slope * (float)(pos - key);
            if (dist_bias) s += dist_bias[(long long)min(pos - key, n_dist - 1) * nh + h];
            sc[j] = s;
            cmax = fmaxf(cmax, s);
        }
        cmax = block_max(cmax, red);
        const float m_new = fmaxf(m, cmax);
        const float corr = expf(m - m_new);          // 0 when m is -inf
        float psum = 0.f;
        for (int j = tid; j < n; j += blockDim.x) {
            const float p = expf(sc[j] - m_new);
            sc[j] = p;
            psum += p;
        }
        psum = block_sum(psum, red);                 // also orders the writes of sc before the reads
        l = l * corr + psum;
        m = m_new;
#pragma unroll
        for (int a = 0; a < 4; ++a) acc[a] *= corr;
        for (int j = 0; j < n; ++j) {
            const int key = c0 + j < n_kept ? c0 + j : lo + (c0 + j - n_kept);
            const TC* vr = vc + paged_offset(cv, seq, key, kvh);
            const float p = sc[j];
#pragma unroll
            for (int a = 0; a < 4; ++a)
                if (tid + 128 * a < hdv) acc[a] = fmaf(p, to_f32<TC>(vr[tid + 128 * a]), acc[a]);
        }
        __syncthreads();
    }
    float inv = out_scale / l;
    if (gate && !gate_wide) inv *= 1.0f / (1.0f + expf(-gate[(long long)t * g_stride + h]));
    TQ* o = out + (long long)t * o_stride + (long long)h * hdv;
    const float* gw = gate && gate_wide ? gate + (long long)t * g_stride + (long long)h * hdv : nullptr;
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int e = tid + 128 * a;
        if (e < hdv) o[e] = from_f32<TQ>(acc[a] * inv * (gw ? 1.0f / (1.0f + expf(-gw[e])) : 1.0f));
    }
}

// q: [T, *] with row stride q_stride (elements), heads side by side; out likewise.
UB_API int ub_attn_simple(const void* q, long long q_stride, int act_dtype, const void* kcache,
                          const void* vcache, int cache_dtype, void* out, long long o_stride,
                          const int* tok_pos, const int* tok_seq, const int* table, int pages_per_seq,
                          int ring, int page, int n_tokens, int nh, int nkv, int hd, int window,
                          float scale, int hd_v, int block, const float* gate, long long g_stride, int keep_first,
                          const float* slopes, int sink, int gate_wide, float out_scale, float softcap,
                          const float* dist_bias, int n_dist, const float* sink_vals, int v_row, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (hd_v <= 0) hd_v = hd;
    if (v_row <= 0) v_row = hd_v;
    if (hd > 1024 || hd <= 0 || hd_v > 512 || v_row < hd_v || nh % nkv != 0 || ring % page != 0 || nh > 65535 || block < 0)
        return UB_ERR_ARG;
    if (dist_bias && n_dist < 1) return UB_ERR_ARG;
    if (keep_first < 0 || (keep_first > 0 && block > 0)) return UB_ERR_ARG;
    PagedKV c{table, pages_per_seq, ring, page, nkv, hd};
    PagedKV cv{table, pages_per_seq, ring, page, nkv, v_row};
    dim3 grid(n_tokens, nh);
    const size_t sm = (size_t)(hd + CHUNK) * sizeof(float);
#define GO(TQ, TC) attn_simple_kernel<TQ, TC><<<grid, 128, sm, st>>>((const TQ*)q, q_stride, (const TC*)kcache, \
        (const TC*)vcache, (TQ*)out, o_stride, tok_pos, tok_seq, c, cv, nh, window, block, gate, g_stride, scale, \
        keep_first, slopes, sink, gate_wide, out_scale, softcap, dist_bias, n_dist, sink_vals, hd_v)
    if (act_dtype == UB_F32 && cache_dtype == UB_F32) GO(float, float);
    else if (act_dtype == UB_BF16 && cache_dtype == UB_BF16) GO(__nv_bfloat16, __nv_bfloat16);
    else if (act_dtype == UB_F32 && cache_dtype == UB_BF16) GO(float, __nv_bfloat16);
    else return UB_ERR_UNSUPPORTED;
#undef GO
    UB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------------
// Placement: from projection rows ``x`` (row stride ldx; the sum of ``n_parts`` parts ``part_stride`` apart) whose
// query heads start at column q_off, key heads at k_off and value heads at v_off, make
//   q_out[t, h, :]   = rotate(norm(q))      activation type, row stride ldq
//   K cache          = rotate(norm(k))      at the token's position
//   V cache          = v                    (head size hd_v)
// norm: RMS over the head with weight qw / kw (null: none); rotate: the first ``rd`` columns in pairs
// (j, j + rd/2) by the token's position (cos, sin [positions, rd/2]; null: none).  k_off < 0: the layer
// has no keys and values of its own and only its queries are made.  gate_out (optional, float32
// [T, nh]) receives the nh columns from g_off on, summed over the parts: one gate a head for the
// attention kernel.  One warp a (token, head).
// ---------------------------------------------------------------------------------------
template <typename TX, typename TQ, typename TC>
__global__ void __launch_bounds__(128)
qkv_place_kernel(const TX* __restrict__ x, long long ldx, int n_parts, long long part_stride, int q_off, int k_off, int v_off,
                 TQ* __restrict__ q_out, long long ldq, const float* __restrict__ qw, const float* __restrict__ kw,
                 const float* __restrict__ cs, const float* __restrict__ sn, int rd, const int* __restrict__ tok_pos,
                 const int* __restrict__ tok_seq, TC* __restrict__ kc, TC* __restrict__ vc, PagedKV c, PagedKV cv,
                 int n_tokens, int nh, float eps, int g_off, float* __restrict__ gate_out) {
    pdl_trigger();
    pdl_wait();
    const int units = nh + (k_off >= 0 ? 2 * c.n_kv_heads : 0);
    const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)n_tokens * units) return;
    const long long t = wid / units;
    const int unit = (int)(wid % units);
    const int pos = tok_pos[t], seq = tok_seq[t];
    auto at = [&](int col) -> float {
        float v = 0.f;
        for (int p = 0; p < n_parts; ++p) v += to_f32<TX>(x[p * part_stride + t * ldx + col]);
        return v;
    };
    if (unit >= nh + c.n_kv_heads) {                       // a value head: copied as it is
        const int g = unit - nh - c.n_kv_heads;
        TC* dst = vc + paged_offset(cv, seq, pos, g);
        for (int e = lane; e < cv.head_dim; e += 32) dst[e] = from_f32<TC>(at(v_off + g * cv.head_dim + e));
        return;
    }
    const bool is_q = unit < nh;
    const int head = is_q ? unit : unit - nh;
    const int hd = c.head_dim;
    if (is_q && gate_out && lane == 0) gate_out[t * nh + head] = at(g_off + head);
    const int c0 = (is_q ? q_off : k_off) + head * hd;
    const float* w = is_q ? qw : kw;
    float v[8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int d = lane + 32 * i;
        v[i] = d < hd ? at(c0 + d) : 0.f;
        ss += v[i] * v[i];
    }
    if (w) {
        ss = warp_sum(ss);
        const float inv = inv_rms(ss, (float)hd, eps);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int d = lane + 32 * i;
            if (d < hd) v[i] *= inv * w[d];
        }
    }
    // the head goes through shared memory so that a lane can reach its rotation partner
    __shared__ float sh[4][256];
    float* my = sh[threadIdx.x >> 5];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) my[d] = v[i];
    }
    __syncwarp();
    const int half = rd >> 1;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int d = lane + 32 * i;
        if (d >= hd) continue;
        float o = v[i];
        if (cs && d < rd) {
            const int j = d < half ? d : d - half;
            const float cj = cs[(long long)pos * half + j], sj = sn[(long long)pos * half + j];
            o = d < half ? my[d] * cj - my[d + half] * sj : my[d] * cj + my[d - half] * sj;
        }
        if (is_q) q_out[t * ldq + (long long)head * hd + d] = from_f32<TQ>(o);
        else kc[paged_offset(c, seq, pos, head) + d] = from_f32<TC>(o);
    }
}

UB_API int ub_qkv_place(const void* x, int x_dtype, long long ldx, int n_parts, long long part_stride, int q_off, int k_off,
                        int v_off, void* q_out, int q_dtype, long long ldq, const float* qw, const float* kw, const float* cs,
                        const float* sn, int rd, const int* tok_pos, const int* tok_seq, void* kcache, void* vcache,
                        int cache_dtype, const int* table, int pages_per_seq, int ring, int page, int n_tokens, int nh,
                        int nkv, int hd, int hd_v, float eps, int g_off, float* gate_out, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (hd <= 0 || hd > 256 || hd_v <= 0 || nh <= 0 || nkv <= 0 || n_parts < 1 || (cs && (rd % 2 || rd < 2 || rd > hd)) ||
        ring % page != 0) return UB_ERR_ARG;
    PagedKV c{table, pages_per_seq, ring, page, nkv, hd};
    PagedKV cv{table, pages_per_seq, ring, page, nkv, hd_v};
    const long long warps = (long long)n_tokens * (nh + (k_off >= 0 ? 2 * nkv : 0));
    const unsigned grid = (unsigned)((warps + 3) / 4);
    cudaError_t e;
#define GO(TX, TQ, TC) e = ub_launch_dependent(qkv_place_kernel<TX, TQ, TC>, dim3(grid), dim3(128), 0, st, (const TX*)x, ldx, n_parts, \
        part_stride, q_off, k_off, v_off, (TQ*)q_out, ldq, qw, kw, cs, sn, rd, tok_pos, tok_seq, (TC*)kcache, (TC*)vcache, c, cv, n_tokens, nh, eps, g_off, gate_out)
    if (x_dtype == UB_F32 && q_dtype == UB_F32 && cache_dtype == UB_F32) GO(float, float, float);
    else if (x_dtype == UB_F32 && q_dtype == UB_BF16 && cache_dtype == UB_BF16) GO(float, __nv_bfloat16, __nv_bfloat16);
    else if (x_dtype == UB_BF16 && q_dtype == UB_BF16 && cache_dtype == UB_BF16) GO(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    else return UB_ERR_UNSUPPORTED;
#undef GO
    return (int)e;
}


// ---------------------------------------------------------------------------------------
// Placement by rows: the same task as above with one block a token, for layers whose norm runs over all
// query heads (and all key heads) of a token at once (``norm_whole``: the weights then have one entry a
// column of the projection, not one a column of a head), whose rotation pairs neighbouring columns
// (``interleaved``: (2j, 2j + 1) instead of (j, j + rd/2)), or whose values are columns of the same row
// taken as they are (v_off may equal k_off: the values are then the keys before norm and rotation).
// gate_out (optional, float32 [T, g_width]) receives the g_width columns from g_off on, summed over parts.
// The token's query and key columns are summed once into shared memory.
// ---------------------------------------------------------------------------------------
template <typename TX, typename TQ, typename TC>
__global__ void __launch_bounds__(256)
qkv_place_rows_kernel(const TX* __restrict__ x, long long ldx, int n_parts, long long part_stride, int q_off, int k_off, int v_off,
                      TQ* __restrict__ q_out, long long ldq, const float* __restrict__ qw, const float* __restrict__ kw,
                      int norm_whole, const float* __restrict__ cs, const float* __restrict__ sn, int rd, int interleaved,
                      const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, TC* __restrict__ kc, TC* __restrict__ vc,
                      PagedKV c, PagedKV cv, int nh, float eps, int g_off, int g_width, float* __restrict__ gate_out) {
    extern __shared__ float row[];                  // [nh * hd] queries, then [nkv * hd] keys
    __shared__ float red[33];
    pdl_trigger();
    pdl_wait();
    const long long t = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = blockDim.x >> 5;
    const int hd = c.head_dim, nkv = k_off >= 0 ? c.n_kv_heads : 0;
    const int qn = nh * hd, kn = nkv * hd;
    const int pos = tok_pos[t], seq = tok_seq[t];
    auto at = [&](int col) -> float {
        float v = 0.f;
        for (int p = 0; p < n_parts; ++p) v += to_f32<TX>(x[p * part_stride + t * ldx + col]);
        return v;
    };
    float sq = 0.f, sk = 0.f;
    for (int i = tid; i < qn + kn; i += blockDim.x) {
        const float v = at(i < qn ? q_off + i : k_off + (i - qn));
        row[i] = v;
        if (i < qn) sq += v * v; else sk += v * v;
    }
    float inv_q = 1.f, inv_k = 1.f;
    if (norm_whole) {
        if (qw) inv_q = inv_rms(block_sum(sq, red), (float)qn, eps);
        if (kw && kn) inv_k = inv_rms(block_sum(sk, red), (float)kn, eps);
    }
    __syncthreads();
    const int half = rd >> 1;
    for (int unit = warp; unit < nh + nkv; unit += n_warps) {
        const bool is_q = unit < nh;
        const int head = is_q ? unit : unit - nh;
        float* my = row + (is_q ? 0 : qn) + head * hd;
        const float* w = is_q ? qw : kw;
        if (w) {
            float inv = is_q ? inv_q : inv_k;
            if (!norm_whole) {
                float ss = 0.f;
                for (int d = lane; d < hd; d += 32) ss += my[d] * my[d];
                inv = inv_rms(warp_sum(ss), (float)hd, eps);
            }
            const float* wh = norm_whole ? w + head * hd : w;
            for (int d = lane; d < hd; d += 32) my[d] *= inv * wh[d];
            __syncwarp();
        }
        for (int d = lane; d < hd; d += 32) {
            float o = my[d];
            if (cs && d < rd) {
                if (interleaved) {
                    const int j = d >> 1;
                    const float cj = cs[(long long)pos * half + j], sj = sn[(long long)pos * half + j];
                    o = (d & 1) ? my[d] * cj + my[d - 1] * sj : my[d] * cj - my[d + 1] * sj;
                } else {
                    const int j = d < half ? d : d - half;
                    const float cj = cs[(long long)pos * half + j], sj = sn[(long long)pos * half + j];
                    o = d < half ? my[d] * cj - my[d + half] * sj : my[d] * cj + my[d - half] * sj;
                }
            }
            if (is_q) q_out[t * ldq + (long long)head * hd + d] = from_f32<TQ>(o);
            else kc[paged_offset(c, seq, pos, head) + d] = from_f32<TC>(o);
        }
    }
    if (k_off >= 0) {
        const int hdv = cv.head_dim;
        for (int i = tid; i < nkv * hdv; i += blockDim.x) {
            const int g = i / hdv, e = i % hdv;
            vc[paged_offset(cv, seq, pos, g) + e] = from_f32<TC>(at(v_off + i));
        }
    }
    if (gate_out)
        for (int i = tid; i < g_width; i += blockDim.x) gate_out[t * g_width + i] = at(g_off + i);
}

UB_API int ub_qkv_place_rows(const void* x, int x_dtype, long long ldx, int n_parts, long long part_stride, int q_off, int k_off,
                             int v_off, void* q_out, int q_dtype, long long ldq, const float* qw, const float* kw, int norm_whole,
                             const float* cs, const float* sn, int rd, int interleaved, const int* tok_pos, const int* tok_seq,
                             void* kcache, void* vcache, int cache_dtype, const int* table, int pages_per_seq, int ring, int page,
                             int n_tokens, int nh, int nkv, int hd, int hd_v, float eps, int g_off, int g_width, float* gate_out,
                             cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (hd <= 0 || hd_v <= 0 || nh <= 0 || nkv <= 0 || n_parts < 1 || (cs && (rd % 2 || rd < 2 || rd > hd)) ||
        ring % page != 0) return UB_ERR_ARG;
    const size_t smem = (size_t)(nh + (k_off >= 0 ? nkv : 0)) * hd * sizeof(float);
    if (smem > 200 * 1024) return UB_ERR_ARG;
    PagedKV c{table, pages_per_seq, ring, page, nkv, hd};
    PagedKV cv{table, pages_per_seq, ring, page, nkv, hd_v};
    cudaError_t e;
#define GO(TX, TQ, TC) do { \
        if (smem > 48 * 1024) cudaFuncSetAttribute(qkv_place_rows_kernel<TX, TQ, TC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        e = ub_launch_dependent(qkv_place_rows_kernel<TX, TQ, TC>, dim3(n_tokens), dim3(256), smem, st, (const TX*)x, ldx, n_parts, \
            part_stride, q_off, k_off, v_off, (TQ*)q_out, ldq, qw, kw, norm_whole, cs, sn, rd, interleaved, tok_pos, tok_seq, \
            (TC*)kcache, (TC*)vcache, c, cv, nh, eps, g_off, g_width, gate_out); } while (0)
    if (x_dtype == UB_F32 && q_dtype == UB_F32 && cache_dtype == UB_F32) GO(float, float, float);
    else if (x_dtype == UB_F32 && q_dtype == UB_BF16 && cache_dtype == UB_BF16) GO(float, __nv_bfloat16, __nv_bfloat16);
    else if (x_dtype == UB_BF16 && q_dtype == UB_BF16 && cache_dtype == UB_BF16) GO(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    else return UB_ERR_UNSUPPORTED;
#undef GO
    return (int)e;
}
