// Linear attention with a per-head decay ("lightning attention"), a recurrence over the tokens of a sequence:
//
//   S_t = a_h S_(t-1) + k_t v_t^T          (S: [dim, vdim] for every head, float32, one a request and layer)
//   o_t = S_t^T q_t
//
// with q, k, v = act(projection) (act = silu or none), read from columns of one wide row in the storage type.
// Everything of the recurrence is float32: the state, the decay (carried as a float32 pair hi + lo so that a
// thousand steps of it do not drift from the constant the model gives), the products and the sums.  The state of a
// request lives in its slot between steps and counts as zero at position 0.
//
// Two forms:
//   * scan: a block walks the rows of one (segment, head, 32 value columns) in order, the state in registers
//     (thread = (value column, an eighth of the key rows)); rows are staged LT_CH at a time.  One row a segment is
//     the decode step.  Every sum has a fixed order, so a row's bits do not depend on how the sequence was cut.
//   * chunked (prompt portions in 16-bit mode): the rows of a segment in chunks of LC rows; within a chunk
//     o = (decay-masked q k^T) v + (a^(i+1) q) S_in, the chunks' own sums U_c = sum_i a^(n-1-i) k_i v_i^T are made
//     in parallel, a short serial pass turns them into the states at the chunks' heads, and the outputs of all chunks
//     are computed in parallel again.
#include "common.cuh"

#define LT_CH 16                 // rows staged at a time by the scan
#define LT_PARTS 8               // warps of a scan block: each owns every eighth key row

template <int ACT> __device__ __forceinline__ float lt_act(float z) {
    return ACT == 0 ? z / (1.0f + expf(-z)) : z;
}

template <typename T, int R, int ACT>
__global__ void __launch_bounds__(32 * LT_PARTS)
lightning_scan_kernel(const T* __restrict__ qkv, int ld, int q_col, int k_col, int v_col, const float* __restrict__ decay_hi,
                      const float* __restrict__ decay_lo, float* __restrict__ state, const int* __restrict__ cu_rows,
                      const int* __restrict__ seg_pos, const int* __restrict__ seg_slot, float* __restrict__ o, int ldo, int H,
                      int dim, int vdim, int write_state) {
    kp_pdl_begin();
    extern __shared__ float lt_sm[];                             // q [LT_CH][dim], k [LT_CH][dim]
    __shared__ float sv[LT_CH][32];
    __shared__ float part[LT_CH][LT_PARTS][32];
    float* sq = lt_sm;
    float* sk = lt_sm + LT_CH * dim;
    const int seg = blockIdx.x, head = blockIdx.y, tile = blockIdx.z;
    const int lane = threadIdx.x & 31, p = threadIdx.x >> 5;
    const int j = tile * 32 + lane;
    const bool jok = j < vdim;
    const float ahi = decay_hi[head], alo = decay_lo[head];
    float* st = state + (((size_t)seg_slot[seg] * H + head) * dim) * vdim;
    float s[R];
    const bool fresh = seg_pos[seg] == 0;
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int i = p + LT_PARTS * r;
        s[r] = (!fresh && jok && i < dim) ? st[(size_t)i * vdim + j] : 0.f;
    }
    const int row0 = cu_rows[seg], row1 = cu_rows[seg + 1];
    for (int t0 = row0; t0 < row1; t0 += LT_CH) {
        const int nt = min(LT_CH, row1 - t0);
        __syncthreads();
        for (int x = threadIdx.x; x < nt * dim; x += blockDim.x) {
            const int t = x / dim, i = x - t * dim;
            const T* row = qkv + (size_t)(t0 + t) * ld + head * dim + i;
            sq[t * dim + i] = lt_act<ACT>(to_f32(row[q_col]));
            sk[t * dim + i] = lt_act<ACT>(to_f32(row[k_col]));
        }
        for (int x = threadIdx.x; x < nt * 32; x += blockDim.x) {
            const int t = x >> 5, l = x & 31, jj = tile * 32 + l;
            sv[t][l] = jj < vdim ? lt_act<ACT>(to_f32(qkv[(size_t)(t0 + t) * ld + v_col + head * vdim + jj])) : 0.f;
        }
        __syncthreads();
        for (int t = 0; t < nt; t++) {
            const float vj = sv[t][lane];
            const float* kt = sk + t * dim;
            const float* qt = sq + t * dim;
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < R; r++) {
                const int i = p + LT_PARTS * r;
                if (i < dim) {
                    s[r] = fmaf(ahi, s[r], fmaf(kt[i], vj, alo * s[r]));
                    acc = fmaf(s[r], qt[i], acc);
                }
            }
            part[t][p][lane] = acc;
        }
        __syncthreads();
        for (int x = threadIdx.x; x < nt * 32; x += blockDim.x) {
            const int t = x >> 5, l = x & 31, jj = tile * 32 + l;
            float sum = part[t][0][l];
#pragma unroll
            for (int q = 1; q < LT_PARTS; q++) sum += part[t][q][l];
            if (jj < vdim) o[(size_t)(t0 + t) * ldo + head * vdim + jj] = sum;
        }
    }
    if (write_state && jok) {
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int i = p + LT_PARTS * r;
            if (i < dim) st[(size_t)i * vdim + j] = s[r];
        }
    }
}

extern "C" {

// qkv: rows [n, ld] in the storage type; q, k at columns q_col, k_col (H heads of dim), v at v_col (H heads of vdim).
// decay_hi + decay_lo: the heads' decays [H].  state: [slots, H, dim, vdim] float32.  o: [n, ldo] float32, heads side by
// side.  act: 0 silu on q, k and v; 1 none.  Segments as everywhere: cu_rows [n_seg + 1], seg_pos, seg_slot [n_seg].
int kp_lightning_scan(const void* qkv, int ld, int q_col, int k_col, int v_col, const float* decay_hi, const float* decay_lo,
                      float* state, const int* cu_rows, const int* seg_pos, const int* seg_slot, float* o, int ldo, int n_seg,
                      int H, int dim, int vdim, int act, int write_state, int dtype, void* stream) {
    if (n_seg <= 0) return 0;
    if (H < 1 || dim < 1 || vdim < 1 || act < 0 || act > 1) return KP_ERR_BAD_ARG;
    if (dim > 32 * LT_PARTS || H > 65535 || (vdim + 31) / 32 > 65535) return KP_ERR_UNSUPPORTED;
    const dim3 grid(n_seg, H, (vdim + 31) / 32), block(32 * LT_PARTS);
    const size_t sm = (size_t)2 * LT_CH * dim * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
#define LT_LAUNCH(T, R, ACT)                                                                                              \
    do {                                                                                                                  \
        if (sm > 28 * 1024) {    /* with the static arrays more than the 48 KB a kernel gets without asking */            \
            cudaError_t e = cudaFuncSetAttribute(lightning_scan_kernel<T, R, ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm); \
            if (e != cudaSuccess) return (int)e;                                                                          \
        }                                                                                                                 \
        kp_launch_pdl(lightning_scan_kernel<T, R, ACT>, grid, block, sm, s, (const T*)qkv, ld, q_col, k_col, v_col, decay_hi, \
                      decay_lo, state, cu_rows, seg_pos, seg_slot, o, ldo, H, dim, vdim, write_state);                    \
    } while (0)
#define LT_BY_R(T, ACT)                                                                                                   \
    do {                                                                                                                  \
        if (dim <= 4 * LT_PARTS) LT_LAUNCH(T, 4, ACT);                                                                    \
        else if (dim <= 8 * LT_PARTS) LT_LAUNCH(T, 8, ACT);                                                               \
        else if (dim <= 16 * LT_PARTS) LT_LAUNCH(T, 16, ACT);                                                             \
        else LT_LAUNCH(T, 32, ACT);                                                                                       \
    } while (0)
    KP_DISPATCH_DTYPE(dtype, T, { if (act == 0) LT_BY_R(T, 0); else LT_BY_R(T, 1); });
#undef LT_BY_R
#undef LT_LAUNCH
    return kp_launch_status();
}

}  // extern "C"
