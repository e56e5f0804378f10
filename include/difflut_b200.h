/*
 * difflut_b200 — C ABI of the B200 (sm_100a) kernels for DiffLUT's LUT-network hot path.
 *
 * Conventions for every entry point
 *   - plain pointers and sizes; all pointers are DEVICE pointers unless a comment says host;
 *   - the caller allocates every input, output and scratch buffer; nothing here allocates,
 *     synchronises or keeps state (exception: the one function documented as such);
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*), in stream order;
 *   - the return value is DL_OK or a negative DL_ERR_* code; the Python shim raises
 *     RuntimeError from it (the reference's bindings raise RuntimeError via TORCH_CHECK,
 *     difflut/nodes/cuda/efd_cuda.cpp:18-40).
 *
 * Layouts
 *   "rows"   row-major (B, F) fp32 — the reference's tensor layout at every API edge.
 *   "t"      feature-major: fp32 [F][Bp] or bit-packed uint32 [F][Bp/32] where bit (b%32) of
 *            word b/32 of row f is sample b of feature f.  Bp = dl_padded_batch(B) (multiple of
 *            128); padded samples hold 0 bits / 0.0 gradients.
 *   tables   DWN: (N, 2^n) fp32, entry index = LUT address, address bit i = node input slot i
 *            (LSB first; difflut/nodes/dwn_node.py:147-153).  A node with several outputs is
 *            passed as several rows that share one row of the index map.
 *   map      (N, n) int32 indices into the layer input (difflut/layers/random_layer.py:195-256).
 */
#ifndef DIFFLUT_B200_H
#define DIFFLUT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* dl_stream_t; /* cudaStream_t */

enum {
    DL_OK = 0,
    DL_ERR_ARG = -1,         /* null pointer, non-positive size, inconsistent sizes      */
    DL_ERR_UNSUPPORTED = -2, /* n outside the supported range of this entry point         */
    DL_ERR_LAUNCH = -3,      /* cudaPeekAtLastError reported a failure after the launch   */
    DL_ERR_ALIGN = -4,       /* a pointer or stride misses the documented alignment       */
    DL_ERR_TOO_LARGE = -5    /* size beyond a documented fixed capacity                   */
};

#define DL_BATCH_ALIGN 128 /* samples; Bp is a multiple of this */
#define DL_MAX_FAST_N 6    /* n <= 6: tables are 64-bit words / 32-lane shuffles */
#define DL_STATIC_SCRATCH_BYTES (16 << 20) /* built-in scratch of dl_dwn_fwd_groupsum_noalloc_t */

int dl_version(void);
const char* dl_error_string(int code);
int64_t dl_padded_batch(int64_t B);

/* ------------------------------------------------------------------ thermometer encoder
 * Replaces ThermometerEncoder.encode (difflut/encoder/thermometer.py:89-116):
 * bit[b, f*T+i] = x[b,f] > thr[f,i] (strict).                                              */

/* rows in, rows out: out (B, F*T) fp32 {0,1} — the reference's exact output tensor. */
int dl_thermo_rows(const float* x, const float* thr, float* out, int64_t B, int64_t F, int64_t T,
                   dl_stream_t stream);
/* rows in, packed feature-major out: bits_t [F*T][Bp/32]. */
int dl_thermo_pack_t(const float* x, const float* thr, uint32_t* bits_t, int64_t B, int64_t F,
                     int64_t T, int64_t Bp, dl_stream_t stream);
/* rows in, packed row-major out: bits (B, ceil(F*T/32)) uint32, bit (c%32) of word c/32. */
int dl_thermo_pack_rows(const float* x, const float* thr, uint32_t* bits, int64_t B, int64_t F,
                        int64_t T, dl_stream_t stream);

/* ------------------------------------------------------------------ layout changes
 * No counterpart in the reference (it keeps fp32 rows everywhere).                         */

/* x (B, F) fp32 rows -> bits_t [F][Bp/32] with bit = x >= threshold (DWN uses 0.5,
 * difflut/nodes/dwn_node.py:147). */
int dl_pack_rows_to_t(const float* x, uint32_t* bits_t, int64_t B, int64_t F, int64_t Bp,
                      float threshold, dl_stream_t stream);
/* fp32 rows (B, F) <-> fp32 feature-major [F][Bp]; padding columns are written as 0. */
int dl_f32_rows_to_t(const float* rows, float* t, int64_t B, int64_t F, int64_t Bp,
                     dl_stream_t stream);
int dl_f32_t_to_rows(const float* t, float* rows, int64_t B, int64_t F, int64_t Bp,
                     dl_stream_t stream);
/* bits_t [F][Bp/32] -> fp32 rows (B, F) of {0,1}. */
int dl_bits_t_to_rows(const uint32_t* bits_t, float* rows, int64_t B, int64_t F, int64_t Bp,
                      dl_stream_t stream);
/* fp32 feature-major [F][ld] (B <= ld valid samples per row) -> bits_t [F][Bp/32], bit = value >=
 * threshold (what dl_pack_rows_to_t does for rows; difflut/nodes/dwn_node.py:147). */
int dl_pack_t_to_t(const float* src_t, uint32_t* bits_t, int64_t F, int64_t B, int64_t ld, int64_t Bp,
                   float threshold, dl_stream_t stream);
/* packed rows (B, Wr) uint32 (bit c%32 of word c/32 = column c) -> bits_t [F][Bp/32]. */
int dl_bits_rows_to_t(const uint32_t* bits_rows, uint32_t* bits_t, int64_t B, int64_t F,
                      int64_t Wr, int64_t Bp, dl_stream_t stream);

/* ------------------------------------------------------------------ RandomLayer gather
 * Replaces mapping_cuda.forward / .backward (difflut/layers/cuda/mapping_cuda.cpp:69-74,
 * kernels difflut/layers/cuda/mapping_cuda_kernel.cu:30-56,136-162):
 * out[b,j,i] = x[b, map[j,i]];  backward gx[b,f] = sum over (j,i) with map[j,i]==f.
 * The backward is a segmented sum over the inverse map (CSR: inv_ptr (F+1), inv_ent holds
 * j*n+i), so it is atomics-free and reproducible.                                          */
int dl_gather_rows(const float* x, const int32_t* map, float* out, int64_t B, int64_t F, int64_t N,
                   int64_t n, dl_stream_t stream);
int dl_gather_rows_bwd(const float* g, const int32_t* inv_ptr, const int32_t* inv_ent, float* gx,
                       int64_t B, int64_t F, int64_t N, int64_t n, dl_stream_t stream);
/* The same sum with the inverse map as a table interleaved by feature: ell[j*F + f] = the j-th column (in
 * ascending order) that feature f collects, -1 once f has no more; max_deg rows.  Gradient rows are staged in
 * shared memory and both streams are read coalesced; N*n must be a multiple of 4 and g 16-byte aligned.  Same
 * order of additions as dl_gather_rows_bwd: same bits. */
int dl_gather_rows_bwd_ell(const float* g, const int32_t* ell, int64_t max_deg, float* gx, int64_t B, int64_t F,
                           int64_t N, int64_t n, dl_stream_t stream);

/* ------------------------------------------------------------------ ConvolutionalLayer patches
 * Replaces nn.Unfold + transpose + view of the convolutional LUT layer
 * (difflut/layers/convolutional.py:170-173,199-205) and its autograd adjoint (fold).
 * x (B, C, H, W) fp32.  A sample is one patch s = b*OH*OW + oy*OW + ox, a feature is
 * f = (c*kh + ki)*kw + kj (nn.Unfold's order); taps in the zero padding read 0.
 * OH = dl_unfold_positions(H, kh, sh, ph), OW likewise (0 = invalid geometry).
 *   dl_unfold_rows     patches (B*OH*OW, C*kh*kw) fp32 rows
 *   dl_unfold_pack_t   bits_t [C*kh*kw][Bp/32], bit = tap >= threshold, Bp >= B*OH*OW a multiple of
 *                      128; samples beyond B*OH*OW pack as 0
 *   dl_fold_rows       gx (B, C, H, W) = adjoint of dl_unfold_rows applied to gpatches (overwritten)
 *   dl_fold_t          the same from a feature-major gradient gpatches_t [C*kh*kw][Bp]
 * The adjoints gather per input pixel (no atomics, fixed summation order).                     */
int64_t dl_unfold_positions(int64_t size, int64_t k, int64_t stride, int64_t pad);
int dl_unfold_rows(const float* x, float* patches, int64_t B, int64_t C, int64_t H, int64_t W,
                   int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw,
                   dl_stream_t stream);
int dl_unfold_pack_t(const float* x, uint32_t* bits_t, int64_t B, int64_t C, int64_t H, int64_t W,
                     int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw,
                     float threshold, int64_t Bp, dl_stream_t stream);
int dl_fold_rows(const float* gpatches, float* gx, int64_t B, int64_t C, int64_t H, int64_t W,
                 int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw,
                 dl_stream_t stream);
int dl_fold_t(const float* gpatches_t, float* gx, int64_t B, int64_t C, int64_t H, int64_t W,
              int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t Bp,
              dl_stream_t stream);

/* ------------------------------------------------------------------ DWN node, feature-major path
 * Together these replace the per-node efd_cuda.forward / .backward calls of a whole layer
 * (difflut/nodes/cuda/efd_cuda.cpp:22-45) and the layer-wide efd_fused_cuda.forward /
 * .backward (difflut/nodes/cuda/efd_fused_cuda.cpp:19-34).  n <= DL_MAX_FAST_N.            */

/* Once per step: tables (N, 2^n) -> efd_t (N, n, 32) and masks (N) uint64.
 * efd_t[j,i,a'] = alpha * sum_k sgn(k_i) * tables[j,k] * beta^popc((a^k) & ~(1<<i)) where a'
 * is the address a with bit i removed (the value does not depend on bit i;
 * difflut/nodes/dwn_node.py:195-227).  Rows a' >= 2^(n-1) are zero.
 * masks[j] bit a = tables[j,a] >= 0.5 (difflut/nodes/dwn_node.py:481).
 * Either output pointer may be null. */
int dl_dwn_prepare(const float* tables, float* efd_t, uint64_t* masks, int64_t N, int64_t n,
                   float alpha, float beta, dl_stream_t stream);
/* The same outputs with an arbitrary weight per Hamming distance instead of beta^h:
 * efd_t[j,i,a'] = scale * sum_k sgn(k_i) * tables[j,k] * w[popc((a^k) & ~(1<<i))].
 * hamming_weights_host is a HOST array of n floats (w[0..n-1]); it is copied at the call.
 * w[h] = 1/(h+1) gives the gradient-stabilised DWN backward
 * (difflut/nodes/dwn_stable_node.py:170-202, kernel difflut/nodes/cuda/dwn_stable_cuda_kernel.cu:80-145). */
int dl_dwn_prepare_weighted(const float* tables, float* efd_t, uint64_t* masks, int64_t N, int64_t n,
                            float scale, const float* hamming_weights_host, dl_stream_t stream);

/* Hard forward on packed bits: out_bits_t[j] = masks[j] looked up at the address formed from
 * rows map[j,0..n-1] of in_bits_t, 32 samples per word at a time (bit-sliced). */
int dl_dwn_fwd_bits_t(const uint32_t* in_bits_t, const int32_t* map, const uint64_t* masks,
                      uint32_t* out_bits_t, int64_t N, int64_t n, int64_t Bp, dl_stream_t stream);

/* Training forward: out_t[j][b] = tables[j, addr(b,j)] (raw value, no clamp;
 * difflut/nodes/dwn_node.py:158).  addr_t [N][Bp] uint8 is optional (null = not written). */
int dl_dwn_fwd_vals_t(const uint32_t* in_bits_t, const int32_t* map, const float* tables,
                      float* out_t, uint8_t* addr_t, int64_t N, int64_t n, int64_t Bp,
                      dl_stream_t stream);

/* Table gradient: gt[j,e] = sum over samples with addr(b,j)==e of g(b,j)
 * (difflut/nodes/dwn_node.py:190-192).  g(b,j) = gscale * g_t[(j / gdiv)][b]: gdiv = 1 reads
 * an [N][Bp] gradient; gdiv = group size reads the [k][Bp] gradient of a following GroupSum
 * without materialising its broadcast.  Overwrites gt.  Also writes addr_t [N][Bp] (the
 * addresses the input-gradient kernel consumes) when addr_t is not null.  Lane-private
 * histograms, fixed summation order: run-to-run reproducible. */
int dl_dwn_bwd_tables_t(const uint32_t* in_bits_t, const int32_t* map, const float* g_t,
                        int64_t gdiv, float gscale, float* gt, uint8_t* addr_t, int64_t N,
                        int64_t n, int64_t Bp, dl_stream_t stream);

/* Input gradient (EFD): gx_t[f][b] = sum over (j,i) with map[j,i]==f of
 * g(b,j) * efd_t[j,i,addr(b,j) without bit i]  (difflut/nodes/dwn_node.py:194-227 followed by
 * the gather's scatter-add, difflut/layers/random_layer.py:301-302), as a segmented sum over
 * the inverse map: inv_ptr (F+1) and inv_ent8, whose entries are (j << 3) | i.  Overwrites gx_t. */
int dl_dwn_bwd_input_t(const uint8_t* addr_t, const float* g_t, int64_t gdiv, float gscale,
                       const float* efd_t, const int32_t* inv_ptr, const int32_t* inv_ent,
                       float* gx_t, int64_t F, int64_t n, int64_t Bp, dl_stream_t stream);
/* The same gradient for a connection map in which every input feature has at most one reader (e.g. the
 * identity map behind a LearnableLayer's soft selection: node j reads features j*n .. j*n+n-1): one warp per
 * (node, 1024 samples) writes the node's n input-gradient rows, gx_t[map[j*n+i]][b]; rows that no node reads
 * are not written.  out_bf16 != 0: gx_t is bf16 [F][Bp] (round to nearest) instead of fp32.  The caller
 * guarantees that the map is disjoint. */
int dl_dwn_bwd_input_disjoint_t(const uint8_t* addr_t, const float* g_t, int64_t gdiv, float gscale,
                                const float* efd_t, const int32_t* map, void* gx_t, int64_t out_bf16, int64_t NO,
                                int64_t n, int64_t Bp, dl_stream_t stream);

/* Fused backward of one layer of a stack (same arithmetic as dl_dwn_bwd_input_t of the layer
 * above followed by dl_dwn_bwd_tables_t of this layer, in one pass).  One warp handles 1024
 * samples of one node f of THIS layer: it forms d(loss)/d(out[f]) either by reading it
 * (inv_ptr == NULL: g(b,f) = gscale_up * g_up[f / gdiv_up][b], e.g. a GroupSum gradient) or by
 * pulling it from the layer above (addr_up [N_up][Bp], g_up, efd_up (N_up, n_up, 32) and the
 * inverse map of the layer above over this layer's nodes, entries (j << 3) | i), then forms this layer's addresses
 * from in_bits_t / map and accumulates the table gradient.  g_out [N][Bp] and addr_out [N][Bp]
 * are written only if not NULL (the first layer of a stack needs neither).
 * gt_partial is caller-provided scratch: dl_dwn_bwd_groups(Bp) slabs of `group_stride` floats
 * (slab g holds the table gradient of samples [1024 g, 1024 (g+1)) at offset f*2^n); sum them
 * with dl_sum_groups, which adds the slabs in order (reproducible).  group_stride == 0: one
 * slab; the kernel itself adds the groups into it in a fixed order (the same warp owns a node in
 * every group), so gt_partial then receives the complete table gradient, reproducible from run to
 * run.  In this mode dl_dwn_bwd_fused_s may keep one histogram over two consecutive 1024-sample
 * blocks (when n == 6, Bp is a multiple of 2048 and there are enough nodes to fill the GPU), which
 * changes the rounding order against the ordered slab sum, not the value.
 * N_up = number of nodes of the layer above (rows of addr_up); ignored when inv_ptr == NULL.   */
int64_t dl_dwn_bwd_groups(int64_t Bp);
int dl_dwn_bwd_fused_t(const uint8_t* addr_up, const float* g_up, int64_t gdiv_up, float gscale_up,
                       const float* efd_up, int64_t n_up, int64_t N_up, const int32_t* inv_ptr,
                       const int32_t* inv_ent, const uint32_t* in_bits_t, const int32_t* map,
                       float* g_out, uint8_t* addr_out, float* gt_partial, int64_t group_stride,
                       int64_t N, int64_t n, int64_t Bp, dl_stream_t stream);
int dl_sum_groups(const float* partial, float* out, int64_t count, int64_t stride, int64_t groups,
                  dl_stream_t stream);

/* ------------------------------------------------------------------ DWN node, materialised-input path
 * Replaces efd_cuda.forward(input, luts) / .backward(input, luts, grad_output, alpha, beta)
 * (difflut/nodes/cuda/efd_cuda.cpp:22-45) for N nodes at once on inputs that are already
 * mapped: xm (B, N, n) fp32 rows (what get_mapping returns,
 * difflut/layers/random_layer.py:258-304 / learnable_layer.py:392-413).
 * tables (N, O, L), out (B, N, O), L = 2^n, n <= 16.                                        */
int dl_dwn_mapped_fwd(const float* xm, const float* tables, float* out, int64_t B, int64_t N,
                      int64_t n, int64_t O, int eval_mode, dl_stream_t stream);
/* gxm (B,N,n) and gt (N,O,L) are overwritten.  efd_full (N, O, L, n) is the full transform
 * written by dl_dwn_prepare_full (caller-provided scratch). */
int dl_dwn_prepare_full(const float* tables, float* efd_full, int64_t NO, int64_t n, float alpha,
                        float beta, dl_stream_t stream);
int dl_dwn_mapped_bwd(const float* xm, const float* g, const float* efd_full, float* gxm,
                      float* gt, int64_t B, int64_t N, int64_t n, int64_t O, dl_stream_t stream);

/* ------------------------------------------------------------------ DWNStable / Hybrid nodes, 6 < n <= 16
 * The n <= 6 forms of these nodes run in the layer kernels (dl_dwn_prepare_weighted + dl_dwn_bwd_*,
 * dl_hybrid_bwd_t).  For wider nodes the forward is dl_dwn_mapped_fwd on the sigmoid-ed tables and the
 * backward restates the reference's per-sample sums on materialised inputs xm (B, N, n):
 *   dl_dwn_stable_mapped_bwd_input  gxm[b,j,i] = scale_j * sum_o g[b,j,o] * sum_k (+-1) table[j,o,k] /
 *                                   (hamming(addr, k without bit i) + 1), sign by bit i of k
 *                                   (difflut/nodes/dwn_stable_node.py:170-202); scale_per_node (N) or NULL
 *                                   and the scalar.  The table gradient is dl_dwn_mapped_bwd's histogram
 *                                   times the scale.
 *   dl_hybrid_mapped_bwd            P[a] = prod_i (a_i ? x_i : 1 - x_i); gt[j,o,a] = sum_b P[a] g[b,j,o];
 *                                   gxm[b,j,i] = sum_o g sum_a table[j,o,a] P[a] (a_i - x_i) /
 *                                   (x_i (1 - x_i) + 1e-8)  (difflut/nodes/hybrid_node.py:160-224).
 *                                   gt (N, O, 2^n) is overwritten (fp32 atomics: not bit-reproducible).    */
int dl_dwn_stable_mapped_bwd_input(const float* xm, const float* tables, const float* g,
                                   const float* scale_per_node, float scale, float* gxm, int64_t B, int64_t N,
                                   int64_t n, int64_t O, dl_stream_t stream);
int dl_hybrid_mapped_bwd(const float* xm, const float* tables, const float* g, float* gxm, float* gt, int64_t B,
                         int64_t N, int64_t n, int64_t O, dl_stream_t stream);

/* ------------------------------------------------------------------ Probabilistic node
 * Replaces probabilistic_cuda.forward(input, raw_weights, temperature) / .backward(...)
 * (difflut/nodes/cuda/probabilistic_cuda.cpp:44-49) for a whole layer, fused with the
 * RandomLayer gather.  Parity target is the reference's PyTorch path
 * (difflut/nodes/probabilistic_node.py:263-300, backward = autograd): no input clamping, input
 * gradient by the product rule (finite at x in {0,1}).
 * x_t [F][Bp] fp32; raw (N, 2^n, O) fp32 (the reference's per-node (2^n, O) tables stacked);
 * outputs are indexed by the virtual node v = j*O + o.  n <= DL_MAX_FAST_N.                  */
int dl_prob_fwd_t(const float* x_t, const int32_t* map, const float* raw, float temperature,
                  float* out_t, int64_t N, int64_t n, int64_t O, int64_t Bp, dl_stream_t stream);
/* Forward fused with the following GroupSum (difflut/utils/modules.py:116-163):
 * logits_t [k][Bp] = (1/tau) * class sums.  `partial` is caller-provided scratch of
 * k*dl_prob_groupsum_splits(N*O,k)*Bp floats; out_t [N*O][Bp] is optional (null = not written). */
int64_t dl_prob_groupsum_splits(int64_t NO, int64_t k);
int dl_prob_fwd_groupsum_t(const float* x_t, const int32_t* map, const float* raw, float temperature,
                           float* out_t, float* partial, float* logits_t, int64_t N, int64_t n,
                           int64_t O, int64_t k, float tau, int64_t Bp, dl_stream_t stream);
/* Backward: graw (N, 2^n, O) (overwritten) and gxm_t [N*n][Bp], the gradient w.r.t. each node's
 * mapped input slot, summed over the node's outputs (overwritten).  g(b,v) = gscale *
 * g_t[v / gdiv][b] as for the DWN kernels.  Either output may be null. */
int dl_prob_bwd_t(const float* x_t, const int32_t* map, const float* raw, float temperature,
                  const float* g_t, int64_t gdiv, float gscale, float* graw, float* gxm_t, int64_t N,
                  int64_t n, int64_t O, int64_t B, int64_t Bp, dl_stream_t stream);
/* Hybrid node backward (difflut/nodes/hybrid_node.py:173-224; replaces hybrid_cuda.backward): the forward
 * is the DWN look-up (dl_dwn_fwd_vals_t), the backward treats the table as a probabilistic node's
 * weights.  tables / gtables (N, O, 2^n) fp32 in the DWN layout (the sigmoid of raw_luts and its
 * chain rule stay with the caller); gtables[j,o,a] = sum_b g * P_a(x_b) (overwritten);
 * gxm_t [N*n][Bp] = the product-rule input gradient times x(1-x)/(x(1-x)+1e-8), summed over the
 * node's outputs (overwritten).  x_t [F][Bp] fp32, g as for dl_prob_bwd_t.  n <= DL_MAX_FAST_N. */
int dl_hybrid_bwd_t(const float* x_t, const int32_t* map, const float* tables, const float* g_t,
                    int64_t gdiv, float gscale, float* gtables, float* gxm_t, int64_t N, int64_t n,
                    int64_t O, int64_t B, int64_t Bp, dl_stream_t stream);
/* gx_t[f][b] = sum over the inverse-map entries e of feature f of src_t[inv_ent[e]][b]: the
 * scatter-add of the gather (difflut/layers/cuda/mapping_cuda_kernel.cu:136-162) as an
 * atomics-free segmented sum in the feature-major layout. */
int dl_seg_sum_t(const float* src_t, const int32_t* inv_ptr, const int32_t* inv_ent, float* gx_t,
                 int64_t F, int64_t Bp, dl_stream_t stream);

/* ------------------------------------------------------------------ LearnableLayer soft connectivity
 * Training path of LearnableMappingModule.forward: softmax(W / tau, dim=-1) followed by
 * x @ S^T (difflut/layers/learnable_layer.py:253-255, which calls F.softmax + torch.matmul), and
 * the two GEMMs + softmax backward autograd derives from it.                                */

/* C (M, N) fp32 = A (M, K) * B (N, K)^T, A and B bf16 row-major (K contiguous), fp32 accumulation in
 * tensor memory (tcgen05.mma fed by TMA).  K must be a multiple of 8.  `status` is one int32 in
 * device memory that the caller zeroes: it stays 0 on success; a non-zero value ((role << 8) |
 * stage) means a bounded wait inside the kernel ran out and C is not valid. */
int dl_gemm_bf16_tn(const void* A, const void* B, float* C, int64_t M, int64_t N, int64_t K, int* status,
                    dl_stream_t stream);
/* The same contraction with the result thresholded and bit-packed in the epilogue instead of stored:
 * bits[m*Wp + n/32] bit n%32 = (C[m][n] >= threshold), the layout and rule of dl_pack_t_to_t applied to the
 * same accumulators (words past N / 32 are not written; Wp*32 >= N).  For consumers that only read
 * "selected value >= 0.5" (DWN nodes behind a LearnableLayer): no fp32 result reaches memory. */
int dl_gemm_bf16_tn_bits(const void* A, const void* B, uint32_t* bits, int64_t M, int64_t N, int64_t K, int64_t Wp,
                         float threshold, int* status, dl_stream_t stream);
/* S = softmax(W / tau) per row of W (M, I), written as bf16 at S_hi[r*ld_out + i]; S_lo (optional)
 * receives bf16(S - S_hi) so that S_hi + S_lo carries 16 mantissa bits. */
int dl_softmax_rows_bf16(const float* W, float tau, void* S_hi, void* S_lo, int64_t ld_out, int64_t M,
                         int64_t I, dl_stream_t stream);

/* Centred single-pass operands of the same contraction: S_c[row, 0..I) = bf16(softmax(W/tau) - 1/I) and
 * S_c[row, ext_col .. ext_col+ext) = 1, 1, 1, 0, ...; dl_row_sum_split_bf16 writes the matching columns of the
 * other operand: A[row, ext_col .. ext_col+ext) = the three-piece bf16 split of scale * sum(A[row, 0..cols)),
 * then zeros (scale = 1/I).  With both, dl_gemm_bf16_tn over K = ext_col + ext gives x . softmax^T with the
 * rounding error of bf16 relative to the deviation from a uniform selection instead of to the weights
 * themselves.  3 <= ext <= 1024; a row pitch that is a multiple of 128 bytes keeps the GEMM's tile loads aligned.  Same reference lines as dl_softmax_rows_bf16. */
int dl_softmax_rows_centered_bf16(const float* W, float tau, void* S_c, int64_t ld_out, int64_t M, int64_t I,
                                  int64_t ext_col, int64_t ext, dl_stream_t stream);
int dl_row_sum_split_bf16(void* A, int64_t ld, int64_t rows, int64_t cols, int64_t ext_col, float scale, int64_t ext,
                          dl_stream_t stream);
/* gW = S * (gS - rowsum(gS * S)) / tau, S recomputed from W in fp32. */
int dl_softmax_bwd_rows(const float* W, const float* gS, float tau, float* gW, int64_t M, int64_t I,
                        dl_stream_t stream);
/* fp32 (rows, cols) -> bf16 at dst[r*ld + c], or transposed at dst[c*ld + r]; dst_lo (optional)
 * receives the bf16 residual. */
int dl_f32_to_bf16(const float* src, void* dst_hi, void* dst_lo, int64_t rows, int64_t cols, int64_t ld,
                   int transpose, dl_stream_t stream);
/* bf16 (rows, cols) with row pitch ld_src -> bf16 (cols, rows) with row pitch ld_dst. */
int dl_bf16_transpose(const void* src, void* dst, int64_t rows, int64_t cols, int64_t ld_src,
                      int64_t ld_dst, dl_stream_t stream);

/* ------------------------------------------------------------------ GroupSum / loss / optimiser
 * GroupSum.forward (difflut/utils/modules.py:116-163): zero-pad F to a multiple of k, class c
 * sums the contiguous block of g = ceil(F/k) columns, divided by tau.                      */
int dl_groupsum_rows(const float* x, float* out, int64_t B, int64_t F, int64_t k, float tau,
                     dl_stream_t stream);
int dl_groupsum_rows_bwd(const float* gout, float* gx, int64_t B, int64_t F, int64_t k, float tau,
                         dl_stream_t stream);
/* feature-major: vals_t [F][Bp] -> logits_t [k][Bp]. */
int dl_groupsum_t(const float* vals_t, float* logits_t, int64_t F, int64_t k, float tau, int64_t Bp,
                  dl_stream_t stream);
/* Fused last layer: logits_t[c][b] = (1/tau) * sum_{j in class c} tables[j, addr(b,j)].
 * `partial` is caller-provided scratch of k*splits*Bp floats (splits from
 * dl_dwn_groupsum_splits); each CTA sums one slice of a class in a fixed order and a second
 * pass adds the slices, so the result is reproducible. */
int64_t dl_dwn_groupsum_splits(int64_t N, int64_t k);
int dl_dwn_fwd_groupsum_t(const uint32_t* in_bits_t, const int32_t* map, const float* tables,
                          float* partial, float* logits_t, int64_t N, int64_t n, int64_t k,
                          float tau, int64_t Bp, dl_stream_t stream);

/* Same result as dl_dwn_fwd_groupsum_t, for hosts that may not allocate device memory.  It has no
 * counterpart in the reference.  Some callers of this library cannot hand it a scratch buffer:
 * an inference server whose device memory was carved up at start-up and belongs to another
 * component, a latency-critical thread that must not pay for cudaMalloc's device-wide
 * synchronisation, or a plain C host with no caching allocator at all.  For them the partial class
 * sums live in a fixed array inside the library (DL_STATIC_SCRATCH_BYTES = 16 MiB, resident on
 * every GPU that loads the library until the process exits); the caller passes only inputs and
 * the logits output.  Limit: k * dl_dwn_groupsum_splits(N, k) * Bp * 4 bytes must fit in that
 * array (the 4000-node, 10-class, 8192-sample case needs 15.6 MiB); anything larger returns
 * DL_ERR_TOO_LARGE and launches nothing.  The first call on a device looks up the array's device
 * address (cudaGetSymbolAddress) and caches it per device; make that first call before starting
 * any stream capture.  No cudaMalloc / cudaFree or other allocating routine is called.  All calls
 * on one GPU share the one array: calls whose kernels can overlap on the GPU (different streams,
 * no ordering between them) race on it and must be serialised by the caller.  Nothing in the
 * array has to be zero on entry - each call overwrites every element it later reads. */
int dl_dwn_fwd_groupsum_noalloc_t(const uint32_t* in_bits_t, const int32_t* map, const float* tables,
                                  float* logits_t, int64_t N, int64_t n, int64_t k, float tau,
                                  int64_t Bp, dl_stream_t stream);

/* ------------------------------------------------------------------ chunk-interleaved bit layout
 * No counterpart in the reference (it has no packed format).  The bit-sliced hard forward
 * (dl_dwn_fwd_bits_t) does not care which sample sits at which bit, while the kernels that need a
 * per-sample table address (dl_dwn_fwd_groupsum_*, dl_dwn_bwd_fused_*) form it for 4 consecutive
 * samples per lane and 128-sample chunk.  In this layout a row has dl_swizzled_words(Bp) =
 * 32 * ceil(Bp/1024) words and, inside each 1024-sample block, bit c + 8r of word w holds sample
 * 128c + 4w + r: a lane's own word then carries its four samples of chunk c one per byte, and an
 * address bit costs one shift and one masked or instead of a shuffle, a shift, a mask, a multiply
 * and two logic ops.  dl_bits_swizzle_t converts natural rows [F][Bp/32] (out of place); run
 * dl_dwn_fwd_bits_t on interleaved rows with Bp rounded up to a multiple of 1024.  The *_s entry
 * points are the *_t ones reading interleaved input bits; every other argument (gradients,
 * addresses, logits) keeps the natural sample order. */
int64_t dl_swizzled_words(int64_t Bp);
/* dl_thermo_pack_t (difflut/encoder/thermometer.py:89-116) writing the interleaved layout directly:
 * bits_s [F*T][dl_swizzled_words(Bp)]. */
int dl_thermo_pack_s(const float* x, const float* thr, uint32_t* bits_s, int64_t B, int64_t F,
                     int64_t T, int64_t Bp, dl_stream_t stream);
int dl_bits_swizzle_t(const uint32_t* bits_t, uint32_t* bits_s, int64_t F, int64_t Bp, dl_stream_t stream);
int dl_dwn_fwd_groupsum_s(const uint32_t* in_bits_s, const int32_t* map, const float* tables,
                          float* partial, float* logits_t, int64_t N, int64_t n, int64_t k, float tau,
                          int64_t Bp, dl_stream_t stream);
/* dl_dwn_fwd_groupsum_s followed by dl_ce_t (loss == NULL) with one launch fewer: the kernel that reduces the
 * partial class sums goes on to the softmax cross-entropy of the 32 samples it holds.  Same bits as the two
 * calls.  k <= 128, else DL_ERR_UNSUPPORTED (nothing launched).  Form the scalar loss with dl_loss_sum. */
int dl_dwn_fwd_groupsum_ce_s(const uint32_t* in_bits_s, const int32_t* map, const float* tables, float* partial,
                             float* logits_t, const int32_t* labels, float* dlogits_t, float* loss_rows, int64_t N,
                             int64_t n, int64_t k, float tau, int64_t B, int64_t B_global, int64_t Bp,
                             dl_stream_t stream);
int dl_dwn_bwd_fused_s(const uint8_t* addr_up, const float* g_up, int64_t gdiv_up, float gscale_up,
                       const float* efd_up, int64_t n_up, int64_t N_up, const int32_t* inv_ptr, const int32_t* inv_ent,
                       const uint32_t* in_bits_s, const int32_t* map, float* g_out, uint8_t* addr_out,
                       float* gt_partial, int64_t group_stride, int64_t N, int64_t n, int64_t Bp,
                       dl_stream_t stream);

/* ------------------------------------------------------------------ layer training options
 * Replace LUTLayerMixin._apply_bit_flip / _apply_gradient_stabilization
 * (difflut/layers/base_layer.py:149-264, 266-339; torch code in the reference).
 *   dl_flip_rows     out[i] = 1 - x[i] with probability p, else x[i] (no gradient: the caller's backward
 *                    is the identity).  Bernoulli per element from a counter-based generator keyed by
 *                    (seed, i).  This is the reference's rule for p >= 0.05 (base_layer.py:189-224).
 *   dl_flip_at       the reference's rule below p = 0.05 (base_layer.py:226-262): exactly `flips` positions
 *                    flip, given by the caller (the first int(count * p) entries of a random permutation of
 *                    the `count` positions, int64, distinct); out = x elsewhere.  out must not alias x.
 *   dl_bits_flip_at_t the same on packed feature-major bits: position e of the row-major (B, F) matrix is
 *                    sample e / F, feature e % F; applied in place with atomic XORs.
 *   dl_bits_flip_t   the same decision per element (f, b) of an (F, B) matrix, applied in place as an XOR to
 *                    packed feature-major bits [F][Bp/32] (flips `x >= 0.5`; differs from thresholding
 *                    1 - x only at x == 0.5 exactly).
 *   dl_grad_rescale  out = (g - mean) * sqrt(target_std / (mean((g - mean)^2) + eps)); mean = 0 unless
 *                    subtract_mean; statistics over the whole (rows, cols) tensor (per_row = 0, needs
 *                    `scratch` of dl_grad_rescale_scratch_doubles() doubles) or per row (per_row = 1).  */
int dl_flip_rows(const float* x, float* out, int64_t count, float probability, int64_t seed,
                 dl_stream_t stream);
int dl_bits_flip_t(uint32_t* bits_t, int64_t F, int64_t B, int64_t Bp, float probability, int64_t seed,
                   dl_stream_t stream);
int dl_flip_at(const float* x, float* out, const int64_t* positions, int64_t count, int64_t flips,
               dl_stream_t stream);
int dl_bits_flip_at_t(uint32_t* bits_t, const int64_t* positions, int64_t flips, int64_t F, int64_t B, int64_t Bp,
                      dl_stream_t stream);
int64_t dl_grad_rescale_scratch_doubles(void);
int dl_grad_rescale(const float* g, float* out, int64_t rows, int64_t cols, int per_row, float target_std,
                    int subtract_mean, float eps, double* scratch, dl_stream_t stream);

/* ------------------------------------------------------------------ data-parallel step over peer memory
 * No counterpart in the reference (it is single-process).  One process per GPU; every rank maps the
 * other ranks' gradient / parameter / flag buffers (CUDA IPC: plain peer pointers) and passes HOST
 * arrays of `world` device pointers, indexed by rank (its own buffer at its own index).
 *   dl_p2p_enable_peer   enable access from the current device to `peer_device` (idempotent)
 *   dl_p2p_barrier       one barrier among the ranks: flags buffers are int32[DL_MAX_PEERS], zeroed
 *                        once; ctrl is a local int32[2] {epoch, status}, zeroed once.  Every wait
 *                        is bounded by timeout_ms; on expiry status becomes 1 + the peer that was
 *                        missing and the kernel returns (the caller reads ctrl[1] when it likes).
 *   dl_p2p_reduce_adam   rank r sums slice r (count/world elements) of all ranks' gradients in
 *                        rank order, applies the Adam step of dl_adam_step to it with its slice-
 *                        sized moments m, v (count/world floats) and stores the new parameters
 *                        into every rank's parameter buffer.  count % (4*world) == 0.  Call
 *                        dl_p2p_barrier before it (gradients complete everywhere) and after it
 *                        (parameters complete everywhere).  ctrl = the barriers' ctrl (or NULL): when
 *                        its status word is non-zero the call changes nothing.                     */
#define DL_MAX_PEERS 8
#define DL_P2P_CHANNELS 8
/*   dl_p2p_exchange_adam the three steps above as ONE kernel, for a slice [offset, offset + count) of the
 *                        flat vector (one layer's tables), so that a layer's exchange can start on a side
 *                        stream as soon as its gradient is complete and travel under the backward of the
 *                        layers below.  flags buffers are int32[DL_P2P_CHANNELS * 2 * DL_MAX_PEERS] (an
 *                        "arrive" and a "done" epoch per channel and peer), ctrl is a local
 *                        int32[1 + 2 * DL_P2P_CHANNELS] {status, then epoch and a CTA counter per channel};
 *                        both zeroed once.  Calls that may overlap in time use different channels.  Rank r
 *                        owns the r-th of `world` equal parts of the slice; its moments m, v hold only its
 *                        parts, the part of this slice at float offset/world (offset and count are
 *                        multiples of 4 * world).  The kernel waits (bounded by timeout_ms) until every
 *                        rank has arrived, reduces, updates and stores its part into every rank's parameter
 *                        buffer, and returns once every rank has done so.  The bias corrections use
 *                        state * beta (this step's powers); with advance_state != 0 the call multiplies
 *                        state by the betas at its end: pass it on the step's last exchange only.  If a
 *                        wait gives up, status becomes 1 + the missing peer and stays so: later calls
 *                        return without touching anything until the host has reset ctrl[0].  A CTA decides
 *                        for itself whether everybody arrived, so a peer that arrives exactly at the limit
 *                        can leave a slice partly updated: a non-zero status invalidates the parameters.
 *                        overlapped != 0: the call runs while a fused backward kernel occupies the GPU on
 *                        another stream; it then launches four-warp CTAs of at most 32 registers per thread,
 *                        which fit beside that kernel's resident CTAs (otherwise they would wait for it to
 *                        end).  overlapped == 0: 256-thread CTAs for a call that has the GPU to itself.
 *                        defer_done != 0: the kernel publishes "done" but does not wait for the peers'; the
 *                        caller then runs dl_p2p_wait_done on the same channel before anything reads the
 *                        parameters or overwrites the gradients again (the start of the next step), which
 *                        takes the second rendezvous off the step's critical path.
 *   dl_p2p_wait_done     waits (bounded) until every peer has published "done" for the channel's latest
 *                        exchange; returns at once before the first exchange.                                */
int dl_p2p_exchange_adam(const void* const* peer_grads_host, const void* const* peer_params_host,
                         const void* const* peer_flags_host, float* m, float* v, double* state, int32_t* ctrl,
                         int64_t offset, int64_t count, int64_t channel, int64_t advance_state, int64_t overlapped,
                         int64_t defer_done, int64_t rank, int64_t world, float lr, float beta1, float beta2, float eps,
                         float gscale, int64_t timeout_ms, dl_stream_t stream);
int dl_p2p_wait_done(const void* const* peer_flags_host, int32_t* ctrl, int64_t channel, int64_t rank, int64_t world,
                     int64_t timeout_ms, dl_stream_t stream);
int dl_p2p_enable_peer(int64_t peer_device);
int dl_p2p_barrier(const void* const* peer_flags_host, int64_t rank, int64_t world, int32_t* ctrl,
                   int64_t timeout_ms, dl_stream_t stream);
int dl_p2p_reduce_adam(const void* const* peer_grads_host, const void* const* peer_params_host, float* m,
                       float* v, double* state, const int32_t* ctrl, int64_t count, int64_t rank, int64_t world,
                       float lr, float beta1, float beta2, float eps, float gscale, dl_stream_t stream);

/* Mean cross-entropy over `B_global` samples of which this call holds B (user code in the
 * reference: nn.CrossEntropyLoss, e.g. tests/test_layers/test_convolutional_learning.py:85-111).
 * logits_t [k][Bp]; labels (B) int32; writes dlogits_t [k][Bp] = (softmax - onehot)/B_global
 * (0 in padding), loss_rows [Bp] per-sample losses and loss[0] = sum(loss_rows)/B_global.
 * loss == NULL skips the sum: dl_loss_sum then forms it from loss_rows, e.g. on another stream, off
 * the path to the backward kernels.  A label outside [0, k) gives that row a zero gradient and a NaN
 * loss (torch's cross_entropy raises for such a label; nothing is read outside the logits here). */
int dl_ce_t(const float* logits_t, const int32_t* labels, float* dlogits_t, float* loss_rows,
            float* loss, int64_t B, int64_t B_global, int64_t k, int64_t Bp, dl_stream_t stream);
int dl_loss_sum(const float* loss_rows, float* loss, int64_t B_global, int64_t Bp, dl_stream_t stream);

/* torch.optim.Adam step (no weight decay / amsgrad) over a flat fp32 tensor.  `state` is a
 * device array of 2 doubles {beta1^t, beta2^t}, initialised to {1, 1}; every call multiplies
 * them on the device first (so a captured CUDA graph can be replayed step after step).
 * g is multiplied by gscale before use (1/world after a sum all-reduce). */
int dl_adam_step(float* p, const float* g, float* m, float* v, double* state, int64_t count,
                 float lr, float beta1, float beta2, float eps, float gscale, dl_stream_t stream);
/* The two halves of dl_adam_step on their own, for a caller that updates slices of the flat vector at
 * different times of a step (each layer's tables as soon as its gradient is complete): dl_adam_advance
 * multiplies the state by the betas (once per step, before the first slice), dl_adam_apply updates one
 * slice with the state as it stands. */
int dl_adam_advance(double* state, float beta1, float beta2, dl_stream_t stream);
int dl_adam_apply(float* p, const float* g, float* m, float* v, const double* state, int64_t count, float lr,
                  float beta1, float beta2, float eps, float gscale, dl_stream_t stream);
/* The same step with the gradient given as `groups` partial slabs of `stride` floats (what
 * dl_dwn_bwd_fused_t writes): g = sum of the slabs in order, also stored to g_out.  Replaces
 * dl_sum_groups + dl_adam_step when no all-reduce sits between them. */
int dl_adam_step_groups(float* p, const float* partial, int64_t stride, int64_t groups, float* g_out,
                        float* m, float* v, double* state, int64_t count, float lr, float beta1,
                        float beta2, float eps, float gscale, dl_stream_t stream);

/* ------------------------------------------------------------------ bit-packed hard-LUT inference
 * The per-layer kernel is dl_dwn_fwd_bits_t.  Class counts of the last layer's packed outputs:
 * counts (B, k) int32, counts[b,c] = number of nodes of class c (contiguous blocks of ceil(N/k))
 * whose output bit is 1 = GroupSum(k, tau=1) of the reference's eval-mode outputs
 * (difflut/nodes/dwn_node.py:457-483, difflut/utils/modules.py:158-163).                   */
int dl_popcount_groupsum_t(const uint32_t* bits_t, int32_t* counts, int64_t N, int64_t k, int64_t B,
                           int64_t Bp, dl_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* DIFFLUT_B200_H */
