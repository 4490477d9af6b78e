// Latent attention: a position's keys and values are kept as ONE small vector c (``rank`` numbers, RMS-normed)
// and one rotated key part (``rot`` numbers) that all heads share.  A head's unrotated key is W_uk c and its value
// W_uv c; the cache holds only [c | rotated part].  Attention then runs in the latent space: a head's query is
// taken through its own W_uk once (q' = W_uk^T q_unrotated, ``rank`` numbers) so that q' . c = q_unrotated . (W_uk c),
// the score is (q' . c + q_rotated . k_rotated) * scale over ONE shared key row of rank + rot numbers, the
// weighted sum of the rows' leading ``rank`` numbers is taken through W_uv afterwards.  This file holds the
// placement kernel; the two small products a head are batched products (gemm_simt.cu; gemm_tcgen05.cu for bfloat16), the
// attention itself is the ordinary attention over one key head whose value rows are the key rows.
//
// latent_place, one block a token, from a projection row x (the float32 sum of ``n_parts`` parts) that holds the
// query heads from column q_off ([dim unrotated | rot rotated] a head) and [rank | rot] latent columns from c_off:
//   q_plain[t, h, :dim]          the unrotated query parts, for the product with W_uk^T
//   q_lat[t, h, rank : rank+rot] the rotated query parts (the leading ``rank`` columns are the product's)
//   cache row of the position    [c / rms(c) * w | rotated key part]
// The rotation turns the pairs (2i, 2i + 1) of the first ``rd`` columns of a rotated part by the position's angles
// (cos, sin [positions, rd / 2], any amplitude already in the tables).
#include "common.cuh"

template <typename TX, typename TQ, typename TC>
__global__ void __launch_bounds__(256)
latent_place_kernel(const TX* __restrict__ x, long long ldx, int n_parts, long long part_stride, int q_off, int c_off,
                    TQ* __restrict__ q_plain, TQ* __restrict__ q_lat, const float* __restrict__ cw, const float* __restrict__ cs,
                    const float* __restrict__ sn, int rd, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                    TC* __restrict__ kc, PagedKV c, int nh, int dim, int rot, int rank, float eps) {
    extern __shared__ float row[];                   // [rank + rot] the latent columns
    __shared__ float red[33];
    pdl_trigger();
    pdl_wait();
    const long long t = blockIdx.x;
    const int tid = threadIdx.x;
    const int pos = tok_pos[t], seq = tok_seq[t];
    const int half = rd >> 1;
    auto at = [&](int col) -> float {
        float v = 0.f;
        for (int p = 0; p < n_parts; ++p) v += to_f32<TX>(x[p * part_stride + t * ldx + col]);
        return v;
    };
    auto turned = [&](float self, float mate, int d) -> float {      // column d of a rotated part; mate: its pair's other column
        const int j = d >> 1;
        const float cj = cs[(long long)pos * half + j], sj = sn[(long long)pos * half + j];
        return (d & 1) ? self * cj + mate * sj : self * cj - mate * sj;
    };
    if (blockIdx.y == 0) {                            // the latent columns: the first block of the token's row of blocks
        float ss = 0.f;
        for (int i = tid; i < rank + rot; i += blockDim.x) {
            const float v = at(c_off + i);
            row[i] = v;
            if (i < rank) ss += v * v;
        }
        ss = block_sum(ss, red);                      // (also orders the writes of row before the reads below)
        const float inv = inv_rms(ss, (float)rank, eps);
        TC* dst = kc + paged_offset(c, seq, pos, 0);
        for (int i = tid; i < rank + rot; i += blockDim.x) {
            float o;
            if (i < rank) o = row[i] * inv * cw[i];
            else {
                const int d = i - rank;
                o = (cs && d < rd) ? turned(row[i], row[rank + (d ^ 1)], d) : row[i];
            }
            dst[i] = from_f32<TC>(o);
        }
    }
    // the query columns, shared out over the token's blocks (a step of few tokens launches several a token)
    const int qd = dim + rot;
    for (int i = blockIdx.y * blockDim.x + tid; i < nh * qd; i += blockDim.x * gridDim.y) {
        const int h = i / qd, d = i % qd;
        const float v = at(q_off + i);
        if (d < dim) { q_plain[(t * nh + h) * dim + d] = from_f32<TQ>(v); continue; }
        const int e = d - dim;
        float o = v;
        if (cs && e < rd) o = turned(v, at(q_off + h * qd + dim + (e ^ 1)), e);
        q_lat[(t * nh + h) * (long long)(rank + rot) + rank + e] = from_f32<TQ>(o);
    }
}

UB_API int ub_latent_place(const void* x, int x_dtype, long long ldx, int n_parts, long long part_stride, int q_off, int c_off,
                           void* q_plain, void* q_lat, int q_dtype, const float* cw, const float* cs, const float* sn, int rd,
                           const int* tok_pos, const int* tok_seq, void* kcache, int cache_dtype, const int* table,
                           int pages_per_seq, int ring, int page, int n_tokens, int nh, int dim, int rot, int rank, float eps,
                           cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (nh <= 0 || dim <= 0 || rot < 0 || rank <= 0 || n_parts < 1 || ring % page != 0 || !cw) return UB_ERR_ARG;
    if (cs && (rd % 2 || rd < 2 || rd > rot)) return UB_ERR_ARG;
    const size_t smem = (size_t)(rank + rot) * sizeof(float);
    if (smem > 48 * 1024) return UB_ERR_ARG;
    PagedKV c{table, pages_per_seq, ring, page, 1, rank + rot};
    cudaError_t e;
    // blocks a token: one for a prompt's many tokens; for few tokens as many as give every thread one query column, up to 16
    const int cols = nh * (dim + rot);
    const int per_token = n_tokens > 64 ? 1 : min(16, max(1, (cols + 255) / 256));
#define GO(TX, TQ, TC) e = ub_launch_dependent(latent_place_kernel<TX, TQ, TC>, dim3(n_tokens, per_token), dim3(256), smem, st, (const TX*)x, ldx, \
        n_parts, part_stride, q_off, c_off, (TQ*)q_plain, (TQ*)q_lat, cw, cs, sn, rd, tok_pos, tok_seq, (TC*)kcache, c, nh, dim, \
        rot, rank, eps)
    if (x_dtype == UB_F32 && q_dtype == UB_F32 && cache_dtype == UB_F32) GO(float, float, float);
    else if (x_dtype == UB_F32 && q_dtype == UB_BF16 && cache_dtype == UB_BF16) GO(float, __nv_bfloat16, __nv_bfloat16);
    else if (x_dtype == UB_BF16 && q_dtype == UB_BF16 && cache_dtype == UB_BF16) GO(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    else return UB_ERR_UNSUPPORTED;
#undef GO
    return (int)e;
}
