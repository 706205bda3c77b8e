/* libresinfer_b200 -- C ABI of the B200 (sm_100a) kernels behind the MEXT / KEXT / ResAttn paths.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (cudaStream_t passed as
 * void*), launches asynchronously on that stream, performs no host synchronisation and returns
 *     0   success,
 *   < 0   arguments rejected (RI_ERR_*); nothing was launched,
 *   > 0   a cudaError_t from the launch.
 * ri_last_error() gives the message of the last failure on the calling thread.  Unless a function
 * says otherwise it allocates nothing: every output and scratch buffer is owned by the caller,
 * like the torch ops these functions replace (ShawRong/ResInfer csrc/bindings/pybind.cpp:28-54:
 * outputs are Tensor(a!) arguments, the ops return ()).
 *
 * File:line citations name the interface of the reference project (ShawRong/ResInfer) that the
 * function stands in for.
 */
#ifndef RESINFER_B200_H_
#define RESINFER_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RI_ABI_VERSION 1

/* error codes (negative returns) */
#define RI_ERR_ARG (-1)
#define RI_ERR_UNSUPPORTED (-2)
#define RI_ERR_DEVICE (-3)
#define RI_ERR_TIMEOUT (-4)

/* input dtypes */
#define RI_DTYPE_BF16 0
#define RI_DTYPE_FP16 1
#define RI_DTYPE_F32 2 /* outputs only: unrounded FP32 result, for accuracy checks */
#define RI_DTYPE_NVFP4 3 /* ri_resattn_decode output only: packed E2M1 codes + E4M3 block scales */

/* FP4 formats */
#define RI_FMT_NVFP4 0 /* 16-element blocks, E4M3 block scale, FP32 global scale */
#define RI_FMT_MXFP4 1 /* 32-element blocks, E8M0 block scale */

/* MEXT output layouts = MExtR1LayoutMode, csrc/nvfp4/cuda/nvfp4_quant_kernels.cu:344-353 */
#define RI_MEXT_CONCAT 0
#define RI_MEXT_ROW_PAIR 1
#define RI_MEXT_TILE8 2
#define RI_MEXT_CONCAT_K 3
#define RI_MEXT_ATTN_TILE8 4
#define RI_MEXT_BASE_ONLY 5 /* this library's addition: base codes [M, K/2] only, no residue */

/* activation layouts the GEMM accepts */
#define RI_GEMM_PLAIN 0    /* act [M, K/2]: y = act . W^T (KEXT: K = K_base + S)            */
#define RI_GEMM_ROW_PAIR 1 /* act [2M, K/2] rows 2i / 2i+1 = base / residue: y_i = sum of both */
#define RI_GEMM_CONCAT_K 2 /* act [M, K] bytes = base | residue along K, W reused for both     */

int ri_abi_version(void);
const char* ri_last_error(void);

/* Number of SMs / compute capability of the current device (cached per device).
 * Returns 0 or an error code. */
int ri_device_info(int* sm_count, int* cc_major, int* cc_minor);

/* NVFP4 MEXT quantiser: x[M,K] (bf16/fp16, row stride in elements) -> base and residue codes plus
 * 128x4-swizzled E4M3 scales in one of the five layouts.
 * gs_inv: device float[n_gs], reciprocal global scale (n_gs == 2: separate residue scale).
 * codes: 2*M'*K/2 bytes (M' = M rounded up to 8 for the tile8 layouts); sf: see the layout rules of
 * csrc/nvfp4/mext.py:151-174 (attn_tile8 expects a zero-filled scale buffer).
 * Replaces torch op nvfp4::scaled_fp4_quant_mext_r1 (csrc/bindings/pybind.cpp:33-37; entry
 * csrc/nvfp4/cuda/nvfp4_quant_kernels.cu:532-612). */
int ri_nvfp4_quant_mext(const void* x, int dtype, int m, int k, int64_t row_stride,
                        const float* gs_inv, int n_gs, uint8_t* codes, int64_t codes_bytes,
                        uint8_t* sf, int64_t sf_bytes, int layout, int enable_pdl, void* stream);

/* NVFP4 KEXT quantiser: base codes of all K channels followed by the residues of the channels
 * selected by mask[K/8] (exactly per8 in {1,2,4} bits set per byte); n_ext = K + K/8*per8.
 * codes [M, n_ext/2]; sf swizzled over n_ext columns, rows up to the next multiple of 128 are
 * written (scale 0).
 * Replaces torch op nvfp4::scaled_fp4_quant (csrc/bindings/pybind.cpp:29-32; entry
 * csrc/nvfp4/cuda/nvfp4_quant_entry.cu:145-186). */
int ri_nvfp4_quant_kext(const void* x, int dtype, int m, int k, int64_t row_stride,
                        const float* gs_inv, const uint8_t* mask, int per8, int n_ext,
                        uint8_t* codes, int64_t codes_bytes, uint8_t* sf, int64_t sf_bytes,
                        int use_swapped_residue, void* stream);

/* ResAttn query quantiser: q[B,Hkv,G,D] bf16 contiguous -> q_pack[B,Hkv,P,D/2] (P = 8 if G == 4
 * else 16; base rows g, residue rows P/2+g; the caller zero-fills q_pack once) and q_sf
 * [B*Hkv*128*D/16] (one private swizzled 128-row tile per (b,hkv)); global scale 1.
 * Replaces torch op nvfp4::scaled_fp4_quant_mext_r1_grouped_q (csrc/bindings/pybind.cpp:38-40;
 * entry csrc/nvfp4/cuda/nvfp4_quant_kernels.cu:655-689). */
int ri_nvfp4_quant_grouped_q(const void* q_bf16, int batch, int num_kv_heads, int group,
                             int head_dim, uint8_t* q_pack, int64_t q_pack_bytes, uint8_t* q_sf,
                             int64_t q_sf_bytes, void* stream);

/* MXFP4 quantiser.  masks == NULL: MEXT, codes [out_rows, K/2] with out_rows = 2M (row_pair) or a
 * multiple of 16 >= 2M (tile8); masks == NULL with per8 == 0 and out_rows == M: plain quantisation
 * without residue (the reference takes that one from FlashInfer, csrc/mxfp4/quantization.py:22-49).  masks != NULL: selective, codes [M, out_row_bytes] with
 * out_row_bytes*2 >= K + K/8*per8 (zero padded).  sf: 128x4-swizzled (swizzle != 0) or linear
 * [out_rows, Ktot/32]; its size must match exactly.  x may be strided (strides in elements).
 * Replaces torch op nvfp4::mxfp4_residue_quant (csrc/bindings/pybind.cpp:41-45; entry
 * csrc/mxfp4/cuda/mxfp4_residue_quant.cu:320-381). */
int ri_mxfp4_quant(const void* x, int dtype, int m, int k, int64_t row_stride, int64_t col_stride,
                   const uint8_t* masks, int per8, uint8_t* codes, int out_rows, int out_row_bytes,
                   uint8_t* sf, int64_t sf_bytes, int swizzle, int tile8, int pdl_mode,
                   void* stream);

/* Block-scaled FP4 GEMM  out[M,N] = alpha * act . W^T  on tcgen05 tensor cores (FP32 accumulate
 * in tensor memory), W [N, K/2] packed codes with row stride w_row_bytes (multiple of 16),
 * scales 128x4-swizzled.  `layout` is one of RI_GEMM_*; K is the weight's K in elements
 * (multiple of 64 for NVFP4, 128 for MXFP4, 256 for RI_GEMM_CONCAT_K).  alpha: device float[n_alpha] (n_alpha == 2, RI_GEMM_ROW_PAIR only:
 * separate factor for the residue term); NULL = 1.0 (MXFP4 has none).
 * The kernel is persistent (one CTA per SM) and cuts the list of (output tile, K tile) units into
 * equal contiguous ranges ("stream-K").  splits: 1 = cut at output-tile boundaries only (no K split,
 * no workspace); 0 = choose; s > 1 = min(tiles * s, SMs) CTAs.  Any plan that splits K needs `workspace`
 * of ri_fp4_gemm_workspace_bytes() bytes (FP32 partials + one ticket per tile), whose first
 * ri_fp4_gemm_counter_bytes() bytes must be zero before the first use (the kernel leaves them zero);
 * the parts of a tile are added in a fixed order, so results are deterministic.
 * out: bf16 or fp16 (or RI_DTYPE_F32) [M, out_row_stride].
 * status: optional device word, set non-zero if a bounded wait inside the kernel expired.
 * Replaces mext_fold_gemm / kext_kloop_gemm_sm100 (csrc/common/fold/sm10x/host.py:190-334), the
 * MXFP4 gemm / fold_gemm (csrc/mxfp4/dense.py:35-66) and the flashinfer.mm_fp4 call of the KEXT
 * route (quant/vllm_integration/residue_linear_op.py:127-137). */
int ri_fp4_gemm(const uint8_t* act, int64_t act_row_bytes, const uint8_t* act_sf,
                int64_t act_sf_bytes, const uint8_t* w, int64_t w_row_bytes, const uint8_t* w_sf,
                int64_t w_sf_bytes, const float* alpha, int n_alpha, void* out, int out_dtype,
                int64_t out_row_stride, int m, int n, int k, int fmt, int layout, int splits,
                void* workspace, int64_t workspace_bytes, int32_t* status, int enable_pdl,
                void* stream);
int64_t ri_fp4_gemm_workspace_bytes(int m, int n, int k, int fmt, int layout, int splits);
int64_t ri_fp4_gemm_counter_bytes(int m, int n);
/* 1 if the plan ri_fp4_gemm chooses for splits == 0 on the current device does not split K
 * (no workspace needed), a value > 1 otherwise. */
int ri_fp4_gemm_auto_splits(int m, int n, int k, int fmt, int layout);

/* ri_fp4_gemm for callers that cannot provide a workspace.  No counterpart in the reference: its
 * GEMMs always take their scratch from the torch caching allocator.  Same arguments and results as
 * ri_fp4_gemm, minus `workspace` / `workspace_bytes`: the K-split scratch is a fixed array of
 * RI_STATIC_SCRATCH_BYTES bytes that is part of the library's device image, so the call never
 * allocates or frees memory.  Meant for callers that gave all free device memory to their own pool
 * at start-up, or whose allocator cannot be reached through the binding.
 *   - A problem whose plan needs more scratch than RI_STATIC_SCRATCH_BYTES (see
 *     ri_fp4_gemm_workspace_bytes) is rejected with RI_ERR_ARG; nothing is launched.
 *   - The array is shared by every call on a device and keeps its last contents; the ticket
 *     counters are cleared on `stream` at the start of each call.  Calls on one device that overlap
 *     in time race on it: order them (one stream, or events).
 *   - The first call on each device looks up the array's device address; make it with the device
 *     that owns `stream` current, and before any stream capture starts. */
#define RI_STATIC_SCRATCH_BYTES (20 * 1024 * 1024)
int ri_fp4_gemm_static_scratch(const uint8_t* act, int64_t act_row_bytes, const uint8_t* act_sf,
                               int64_t act_sf_bytes, const uint8_t* w, int64_t w_row_bytes,
                               const uint8_t* w_sf, int64_t w_sf_bytes, const float* alpha, int n_alpha,
                               void* out, int out_dtype, int64_t out_row_stride, int m, int n, int k,
                               int fmt, int layout, int splits, int32_t* status, int enable_pdl,
                               void* stream);

/* One-shot all-reduce (sum) of a small BF16 tensor over peer memory, for the partial outputs of row-parallel
 * linears in a tensor-parallel decode step on one node.  Stands where the reference relies on vLLM's
 * RowParallelLinear all-reduce after its rank-local linear (`apply` of quant/vllm_integration/
 * linear_method_v2.py and linear_method_mxfp4.py returns the partial).
 *   rank_data[r]   this process's mapping of rank r's partial (`numel` BF16 values, 16-byte aligned; for
 *                  r == rank the local buffer itself); the partial must have been written by earlier work on
 *                  `stream`
 *   rank_flags[r]  this process's mapping of rank r's flag array (ri_peer_allreduce_flag_bytes() bytes,
 *                  zeroed once before the first call, owned by this library afterwards)
 *   state          local device memory, ri_peer_allreduce_state_bytes() bytes, zeroed once
 *   out            local result, `numel` BF16 values, 16-byte aligned, not one of the mapped partials
 * Every rank of the group must make the same sequence of calls.  A rank's partial buffer may be
 * overwritten again after its NEXT call of this function has completed (alternate between two
 * buffers).  The wait for the peers is bounded (ten seconds unless ri_peer_allreduce_set_wait_ms
 * says otherwise; measured on the GPU's nanosecond timer); on expiry `status` (optional) receives
 * 0x40000000 | missing_rank << 8 | rank and `out` receives this rank's own partial -- a defined value,
 * not the sum -- so callers must look at the status word where that matters.  The sum is taken in
 * rank order with FP32 accumulation, so every rank holds the same bits.  When more than 4 MB would have to be
 * read from the peers (more than two ranks), each rank sums only its own slice of the vectors, writes the sums back
 * into its own partial buffer and fetches the other slices from their owners after a second hand-shake -- same bits,
 * 2 (world - 1) / world instead of (world - 1) times the bytes; the partial buffer then holds those sums in this
 * rank's slice afterwards.  enable_pdl != 0 launches
 * with programmatic stream serialisation: the kernel's launch overlaps the tail of the kernel that
 * wrote the partial and its first instruction waits for that kernel's completion. */
int64_t ri_peer_allreduce_flag_bytes(void);
int64_t ri_peer_allreduce_state_bytes(void);
void ri_peer_allreduce_set_wait_ms(int milliseconds);
int ri_peer_allreduce_bf16(const void* const* rank_data, void* const* rank_flags, int rank, int world,
                           int64_t numel, void* out, void* state, int32_t* status, void* stream,
                           int enable_pdl);

/* ri_fp4_gemm of a row-parallel linear with the all-reduce of the BF16 partial outputs done by the same kernel
 * over peer memory.  The reference returns the rank-local partial from its linear methods and leaves the sum to
 * vLLM's RowParallelLinear (quant/vllm_integration/linear_method_v2.py, linear_method_mxfp4.py; the partition rule
 * is quant/vllm_integration/residue_tp.py); this entry point is that pair of steps in one launch.
 *   rank_inboxes[r]   this process's mapping of rank r's inbox: `world` areas of 4 * inbox_area bytes, area s
 *                     receiving rank s's partial ([M, partial_row_stride] BF16 in the first half of the area, or
 *                     the pair format below in all of it); 16-byte aligned; for r == rank the local inbox
 *   rank_flags[r]     this process's mapping of rank r's flag array, ri_fp4_gemm_allreduce_flag_bytes(max_tiles)
 *                     bytes, zeroed once before the first call and owned by the library afterwards
 *   tile_calls        local device memory, ri_fp4_gemm_allreduce_call_bytes(max_tiles) bytes, zeroed once
 *   max_tiles         flag entries the arrays hold; a call needs at most ri_fp4_gemm_allreduce_tiles(M, N)
 *   reduced_out       local result [M, reduced_row_stride] BF16, not part of an inbox
 * The CTA that completes a 128-column output tile goes over the tile twice.  First pass: the BF16 tile is stored
 * into this rank's area of every PEER's inbox (plain 16-byte stores that cross NVLink without waiting for
 * anything) and the tile's call number is published to every peer with a system-scope release.  After the wait for
 * the peers' announcements of the same tile, second pass: the tile is formed again from tensor memory (or the
 * K-split partials), the peers' tiles are read from the local inbox, everything is added in rank order in FP32
 * and written as BF16.  Every rank holds the same bits, and they equal ri_fp4_gemm followed by
 * ri_peer_allreduce_bf16.  No multicast, no NCCL, no load from a peer; this rank's own tile never travels through
 * memory (its area of the local inbox stays unused).
 * Small partials (ri_fp4_gemm_allreduce_uses_pairs(M, N, world): at most 2 MiB leave a rank per call) use neither
 * the flag arrays nor any fence: every 32-bit word travels as an aligned 8-byte pair (word, call number), the
 * reader polls the pairs of the vector it needs until all carry this call's number.  The call number counts the
 * launches on these inboxes (two words behind the per-tile counts in tile_calls; the last CTA of a launch adds one).
 * Every rank must make the same sequence of calls with the same shapes and `splits`; an inbox may be written
 * again after the rank's NEXT fused call has completed (alternate between two inboxes).  The wait is bounded as
 * for ri_peer_allreduce_bf16 (ri_peer_allreduce_set_wait_ms); on expiry `status` receives
 * 0x40000000 | missing_rank << 8 | rank, the tile of reduced_out receives this rank's own partial, and the flag
 * arrays and call counters of all ranks must be zeroed together before the next call.  The other arguments are
 * ri_fp4_gemm's; N, both row strides and inbox_area must be multiples of 8. */
int64_t ri_fp4_gemm_allreduce_tiles(int m, int n);
int ri_fp4_gemm_allreduce_uses_pairs(int m, int n, int world);
int64_t ri_fp4_gemm_allreduce_flag_bytes(int64_t max_tiles);
int64_t ri_fp4_gemm_allreduce_call_bytes(int64_t max_tiles);
int ri_fp4_gemm_allreduce(const uint8_t* act, int64_t act_row_bytes, const uint8_t* act_sf,
                          int64_t act_sf_bytes, const uint8_t* w, int64_t w_row_bytes, const uint8_t* w_sf,
                          int64_t w_sf_bytes, const float* alpha, int n_alpha, int64_t partial_row_stride,
                          int m, int n, int k, int fmt, int layout, int splits, void* workspace,
                          int64_t workspace_bytes, int32_t* status, int enable_pdl, void* stream,
                          void* const* rank_inboxes, int64_t inbox_area, void* const* rank_flags,
                          void* tile_calls, int64_t max_tiles, int rank, int world, void* reduced_out,
                          int64_t reduced_row_stride);

/* ResAttn: residue-compensated paged NVFP4-KV decode attention, one query token per sequence.
 * q [B,Hq,D] bf16; k_data/v_data [pages,Hkv,page_size,D/2]; k_sf/v_sf [pages,Hkv,page_size,D/16]
 * E4M3 bytes (linear); block_tables int32 [B, bt_stride]; seq_lens int32 [B]; out [B,Hq,D] bf16
 * (out_dtype RI_DTYPE_BF16; RI_DTYPE_F32 writes the unrounded result; RI_DTYPE_NVFP4 writes the
 * activation format of the following projection: `out` = uint8 codes [B, Hq*D/2], out_block_scale =
 * 128x4-swizzled E4M3 scales over rows = sequences and hidden = Hq*D, scale = e4m3(amax * g / 6) with
 * g = *out_global_scale -- quantize_nvfp4_block16 / output_scale_offset, csrc/resattn/output.py:10-34,
 * run_paged_fp4_decode_qmul4_tmem_nvfp4, quant/vllm_integration/attn/decode.py:55-101).
 * score_scale = sm_scale * k_global_scale, out_scale = v_global_scale.  The query is quantised
 * to NVFP4 + NVFP4 residue inside the kernel (q_residue == 0 drops the residue rows); q_pack / q_sf
 * are optional (NULL) outputs that receive the quantised query in the layout of
 * ri_nvfp4_quant_grouped_q.  page_size is a multiple of 16.  splits > 1 cuts the KV range into
 * `splits` pieces of ceil(ceil(max_kv_len / 128) / splits) 128-token tiles each -- the same piece
 * size for every sequence, so long sequences use many splits and short ones few (CTAs of unused
 * splits leave at once) -- and uses `workspace` (ri_resattn_workspace_bytes) for the per-split
 * partial (o, l, m).  The merge is part of the same launch: every CTA takes a ticket per (sequence,
 * KV head) and the one that draws the last ticket sums the partials in split order (deterministic;
 * the reference's fused reducer spins instead, csrc/resattn/kernel_paged_decode.py:2365-2431).  The
 * first ri_resattn_counter_bytes(batch, num_q_heads) bytes of the workspace are those tickets: they
 * must be zero before the first call and the kernel leaves them zero, so a workspace may be reused
 * by calls that do not overlap on the GPU.  max_kv_len: upper bound of seq_lens
 * for this call (0 = what the block table can hold, bt_stride * page_size).  status: optional
 * device word, set non-zero if a bounded wait inside the kernel expired.
 * Replaces run_paged_fp4_decode_qmul4_tmem (csrc/resattn/host.py:489-606). */
int ri_resattn_decode(const void* q_bf16, const uint8_t* k_data, const uint8_t* k_sf,
                      const uint8_t* v_data, const uint8_t* v_sf, int64_t num_pages,
                      const int32_t* block_tables, int64_t bt_stride, const int32_t* seq_lens,
                      int batch, int num_q_heads, int num_kv_heads, int head_dim, int page_size,
                      int max_kv_len, float score_scale, float out_scale, void* out, int out_dtype, uint8_t* q_pack,
                      int64_t q_pack_bytes, uint8_t* q_sf, int64_t q_sf_bytes,
                      const float* out_global_scale, uint8_t* out_block_scale, int64_t out_block_scale_bytes,
                      int splits, void* workspace, int64_t workspace_bytes, int q_residue, int32_t* status,
                      void* stream);
/* How the partial results of the KV splits of one (sequence, KV head) are combined -- in both cases inside the
 * decode launch, in split order, with identical results (the reference's reducers: csrc/resattn/plan.py:36-92,
 * kernel_paged_decode.py:80-104).
 * TICKET:  partials go through the workspace; the CTA that draws the last ticket combines them ("kernel" /
 *          "gmem_fused" of the reference).  Any split count, any output type.
 * CLUSTER: the splits are one thread-block cluster and combine through distributed shared memory, each CTA a share
 *          of the output ("cga_sharded" of the reference).  2 to 8 or 16 splits, BF16 / FP32 output, no workspace;
 *          meant for grids of a few clusters (one sequence, or a tensor-parallel shard's few KV heads): measured on
 *          B200 it is a fifth faster than TICKET there and slower from about sixteen clusters up. */
#define RI_ATTN_REDUCER_TICKET 0
#define RI_ATTN_REDUCER_CLUSTER 1

/* ri_resattn_decode with the reducer as an argument, over a pool whose pages need not be packed back to back: `code_page_stride` / `sf_page_stride` are
 * the bytes from one page's [Hkv, page_size] rows of codes / block scales to the next page's (multiples of 16;
 * 0 = dense), the same for K and V.  This is the form vLLM's NVFP4 cache has -- every page keeps K codes | K scales
 * | V codes | V scales together, and the reference hands its kernel strided views of it
 * (quant/vllm_integration/attn/backend.py:125-144) -- so the cache is read in place, no repacking. */
int ri_resattn_decode_strided(const void* q_bf16, const uint8_t* k_data, const uint8_t* k_sf,
                              const uint8_t* v_data, const uint8_t* v_sf, int64_t num_pages,
                              int64_t code_page_stride, int64_t sf_page_stride,
                              const int32_t* block_tables, int64_t bt_stride, const int32_t* seq_lens,
                              int batch, int num_q_heads, int num_kv_heads, int head_dim, int page_size,
                              int max_kv_len, float score_scale, float out_scale, void* out, int out_dtype, uint8_t* q_pack,
                              int64_t q_pack_bytes, uint8_t* q_sf, int64_t q_sf_bytes,
                              const float* out_global_scale, uint8_t* out_block_scale, int64_t out_block_scale_bytes,
                              int splits, int reducer, void* workspace, int64_t workspace_bytes, int q_residue,
                              int32_t* status, void* stream);
/* Sets the launch attributes of the decode kernel's instantiations for `head_dim` on the current device, which the
 * first ri_resattn_decode would otherwise do.  The reference compiles its kernel variants at run time and lists the
 * compilations for vLLM's warm-up (quant/vllm_integration/attn/warmup.py:21-44); this is what is left of that step
 * when the kernels are built ahead of time. */
int ri_resattn_prepare(int head_dim);
/* Number format of V and P in the second product of ri_resattn_decode, process-wide: 0 (default) = FP16 -- code x
 * block scale is exact in FP16 and P keeps 11 bits, 3e-3 from exact attention; 1 = E4M3 for both, the reference's
 * choice (csrc/resattn/kernel_paged_decode.py:1958-1963, csrc/resattn/qmul4.py:45): tcgen05.mma kind::f8f6f4,
 * half the shared-memory bytes per tile and a third copy stage, about 3e-2 from exact attention, and V saturates
 * at 448 (caches whose code x block scale products stay in the FP8 range). */
void ri_resattn_set_pv_format(int e4m3);
int ri_resattn_get_pv_format(void);
int64_t ri_resattn_workspace_bytes(int batch, int num_q_heads, int head_dim, int splits);
int64_t ri_resattn_counter_bytes(int batch, int num_q_heads);

/* Test helper: out[i] = rcp.approx.ftz.f32(in[i]) on the device (the quantisers' reciprocal). */
int ri_rcp_approx(const float* in, float* out, int n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* RESINFER_B200_H_ */
