/*
 * glow_b200 -- C ABI of the B200 (sm_100a) kernels behind pytorch/glow's quantized
 * inference hot path.
 *
 * Every entry point is the device-side counterpart of one `extern "C" libjit_*` kernel that
 * Glow's CPU backend calls from JIT-ed code (or of one Interpreter `fwd*Inst` where the CPU
 * backend has none); the comment on each names the reference interface it replaces.  The
 * argument meaning is the reference's, with these changes that hold for all of them:
 *   - every tensor pointer is a DEVICE pointer (the caller owns all buffers; the library
 *     allocates nothing -- scratch memory is passed in as `workspace`);
 *   - dims are passed as int64 scalars instead of `dim_t*` arrays;
 *   - `stream` is a cudaStream_t (as void*); all work is enqueued on it, nothing synchronises;
 *   - `status` (may be NULL) is a device int32 that kernels OR the GLOWB200_STATUS_* bits
 *     into when they meet invalid input; the kernel still returns normally and skips the
 *     offending element (libjit itself does no bounds checks; the rules are those of Glow's
 *     lib/Runtime/InputSanitizer.cpp:31-110);
 *   - the int return value is GLOWB200_OK or a GLOWB200_ERR_* code for argument / launch
 *     errors detected on the host; glowb200_last_error() gives the message.  No exceptions
 *     cross this boundary.
 * Entry points are re-entrant; calls on one stream are ordered.
 */
#ifndef GLOW_B200_H
#define GLOW_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GLOWB200_OK 0
#define GLOWB200_ERR_INVALID_ARGUMENT 1
#define GLOWB200_ERR_UNSUPPORTED 2
#define GLOWB200_ERR_WORKSPACE_TOO_SMALL 3
#define GLOWB200_ERR_CUDA 4

/* Codes returned by the host runtime (glowb200_function_* / glowb200_device_manager_*), named
 * after glow::ErrorValue::ErrorCode (include/glow/Support/Error.h:292-339). */
#define GLOWB200_RUNTIME_ERROR 101
#define GLOWB200_RUNTIME_OUT_OF_DEVICE_MEMORY 102
#define GLOWB200_RUNTIME_NET_NOT_FOUND 103
#define GLOWB200_RUNTIME_DEVICE_NONRECOVERABLE 104

/* Bits OR-ed into *status by kernels. */
#define GLOWB200_STATUS_INDEX_OUT_OF_RANGE 1 /* an index outside [0, rows): that row is skipped   */
#define GLOWB200_STATUS_LENGTHS_OVERRUN 2    /* sum(lengths) > len(indices): bags are truncated   */
#define GLOWB200_STATUS_NEGATIVE_LENGTH 4    /* a negative length: treated as 0                   */
#define GLOWB200_STATUS_BAD_OFFSETS 8        /* offsets not monotone / out of range: bag is empty */
#define GLOWB200_STATUS_WAIT_TIMEOUT 16      /* a bounded device-side wait gave up                */
#define GLOWB200_STATUS_UNSUPPORTED_TABLE 32 /* split-embedding table of an unsupported type; a   */
                                             /* dynamic-FC row whose zero point is not 0          */

/* Fused-rowwise table kinds (glow::ElemKind, include/glow/Base/Type.h:424-433).  A row is the
 * quantized payload followed by scale then offset (include/glow/Base/Tensor.h:1585-1607). */
#define GLOWB200_UINT8_FUSED 0      /* UInt8FusedQTy:     D bytes   + fp32 scale + fp32 offset */
#define GLOWB200_UINT8_FUSED_FP16 1 /* UInt8FusedFP16QTy: D bytes   + fp16 scale + fp16 offset */
#define GLOWB200_UINT4_FUSED 2      /* UInt4FusedQTy:     D/2 bytes + fp32 scale + fp32 offset */
#define GLOWB200_UINT4_FUSED_FP16 3 /* UInt4FusedFP16QTy: D/2 bytes + fp16 scale + fp16 offset */

typedef void *glowb200_stream_t;

/* Message of the last error returned on this host thread ("" if none). */
const char *glowb200_last_error(void);
/* Library version string. */
const char *glowb200_version(void);

/* Programmatic dependent launch.  The library launches its contraction, convolution-preparation and
 * NHWC element-wise kernels so that a kernel may set up (barriers, tensor memory) beside the tail of
 * the kernel before it in the stream; it touches global memory only after that kernel has completed
 * (griddepcontrol.wait), so results do not change.  A kernel that waits this way holds its shared
 * memory and thread slots: a caller that runs another stream beside it (Glow's executor running two
 * partitions on one device) may prefer ordinary launches for that stream.  enabled: 1 on, 0 off,
 * -1 back to the default (on, unless the environment has GLOWB200_PDL=0).  Process-wide; takes
 * effect for the launches (or CUDA-graph captures) that follow.  Returns the previous state (0 / 1). */
int glowb200_set_programmatic_launch(int enabled);

/* ---------------------------------------------------------------------------------------
 * Embedding gather-pool
 * ------------------------------------------------------------------------------------- */

/* One table's worth of work in a batched launch (all pointers are device pointers).
 * Alignment: `data` must start on a 16-byte boundary (any offset of a cudaMalloc'ed slab that
 * keeps Glow's 64-byte tensor alignment does); weights, indices and lengths on the boundary of
 * their element type.  The batched entry points read the descriptors on the device and use
 * vector loads on the strength of this -- a misaligned table is not detected, it faults.
 * `segments` must not exceed the max_segments the launch is given: surplus bags are left out
 * and reported through GLOWB200_STATUS_BAD_OFFSETS. */
typedef struct glowb200_slws_job {
  const void *data;       /* fused table [rows, in_line_size] bytes                         */
  const void *weights;    /* per-index weights, the result's element type, [num_indices]     */
  const void *indices;    /* int32 or int64 [num_indices]                                    */
  const int32_t *lengths; /* [segments]                                                      */
  void *dest;             /* result, row i at dest + i * dest_stride elements                */
  int64_t rows;           /* table rows (for the index range check)                          */
  int64_t num_indices;    /* entries readable in indices / weights                           */
  int64_t dest_stride;    /* elements between consecutive result rows (>= out_line_size)     */
  int64_t segments;       /* number of bags                                                  */
  /* Optional scatter of the bags over several destination buffers -- the pooled-embedding
   * exchange of a table-sharded model done by the pooling kernel itself: when bags_per_dest > 0,
   * bag b is written to row b % bags_per_dest of dests[b / bags_per_dest] instead of `dest`.
   * `dests` is a DEVICE array of pointers, which may address other GPUs' memory (see
   * glowb200_peer_buffer_*); the stores are ordinary peer stores. */
  void *const *dests;
  int64_t bags_per_dest;
  /* Row-range sharding of one table over several GPUs: `data` holds the table's rows
   * [row_begin, row_begin + rows) and the indices are numbers of the whole table, which has
   * global_rows rows.  An index inside the whole table but outside this shard is skipped
   * silently (another shard pools it); the result is this shard's partial sum.  Honoured by
   * glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum_row_sharded only; every other
   * entry point takes the table as whole. */
  int64_t row_begin;
  int64_t global_rows;
} glowb200_slws_job;

/* Bytes of scratch the gather-pool entry points need for `num_jobs` tables of at most
 * `max_segments` bags each (segment start offsets, one int64 array per table). */
size_t glowb200_slws_workspace_bytes(int64_t max_segments, int64_t num_jobs);

/* FusedRowwiseQuantizedSparseLengthsWeightedSum.
 * Replaces libjit_fused_rowwise_quantized_sparse_lengths_weighted_sum_f_u / _f_i32 / _f
 * (lib/LLVMIRCodeGen/libjit/libjit.cpp:2416-2452, generic body :1253-1276; call emitted at
 * lib/LLVMIRCodeGen/LLVMIRGen.cpp:3638-3659) for UInt8FusedQTy, and
 * BoundInterpreterFunction::fwdFusedRowwiseQuantizedSparseLengthsWeightedSumInst
 * (lib/Backends/Interpreter/InterpreterNodes.cpp:5764-5889) for the other three kinds.
 *   dest [segments, out_line_size] fp32, or fp16 when out_is_fp16; weights have dest's type;
 *   data [rows, in_line_size] bytes of `kind`; lengths int32 [segments];
 *   use_fp16_accumulation as the node flag (honoured only for an fp16 result on an
 *   fp16-scale table, like the reference's dispatcher).
 *   in_line_size may exceed the bytes out_line_size columns and the scale/offset pair need:
 *   the pair is the last bytes of the row, the bytes between are padding
 *   (see glowb200_fused_rows_pad).
 * The unweighted FusedRowwiseQuantizedSparseLengthsSum is this call with weights of 1
 * (lib/Optimizer/Lower/Lower.cpp:1590-1606). */
int glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum(
    void *dest, const void *data, int kind, int64_t rows, const void *weights, const void *indices,
    int indices_are_int64, const int32_t *lengths, int64_t segments, int64_t num_indices,
    int64_t in_line_size, int64_t out_line_size, int out_is_fp16, int use_fp16_accumulation,
    void *workspace, size_t workspace_bytes, int32_t *status, glowb200_stream_t stream);

/* The same operator for small requests where latency counts: every bag gets a whole warp (the
 * thread mapping the entry point above gives tables with very uneven bags), so a bag's rows are
 * fetched together instead of four at a time -- the launch of benchmark configuration 1 (1024
 * bags of about 32 rows) takes a quarter of the time; up to 2048 bags the warps also add up the
 * lengths before their bag themselves, so the request is a single launch.  fp32 accumulation only.  The rows of a bag
 * are summed in another order than above: results agree within the operator's tolerance (1e-5
 * relative) but are not bit-identical to the other entry points', which is why the choice is the
 * caller's and not made from the size of the launch. */
int glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum_low_latency(
    void *dest, const void *data, int kind, int64_t rows, const void *weights, const void *indices,
    int indices_are_int64, const int32_t *lengths, int64_t segments, int64_t num_indices,
    int64_t in_line_size, int64_t out_line_size, int out_is_fp16, void *workspace,
    size_t workspace_bytes, int32_t *status, glowb200_stream_t stream);

/* The same operator over `num_jobs` tables of one kind and one row width in ONE launch
 * (how Glow's SLS benchmark and the SparseNN partitioner present many tables to a device:
 * tests/benchmark/SLSBench.cpp:49-104, lib/Partitioner/Partitioner.cpp:1611-1685).
 * `jobs` is a DEVICE array of `num_jobs` descriptors; `max_segments` bounds jobs[i].segments.
 * dest_stride lets every table write its bags straight into a wider row (a concatenated
 * [batch, tables*D] activation or a per-peer send buffer). */
int glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum_batched(
    const glowb200_slws_job *jobs, int64_t num_jobs, int64_t max_segments, int kind,
    int indices_are_int64, int64_t in_line_size, int64_t out_line_size, int out_is_fp16,
    int use_fp16_accumulation, void *workspace, size_t workspace_bytes, int32_t *status,
    glowb200_stream_t stream);

/* The batched operator over row-range SHARDS of tables (row_begin / global_rows of every
 * descriptor are honoured): each launch gives the fp32 partial sums of the rows this GPU holds;
 * weights and dest are fp32 for every kind (an fp16 weight widened is the same number), and
 * glowb200_sum_partials adds the shards' results and rounds once to the result type.  No
 * reference counterpart: Glow does not split an embedding table by rows
 * (ParallelTransformKind splits SparseLengthsSum by batch only,
 * lib/Optimizer/GraphOptimizer/GraphOptimizer.cpp:7263-7300). */
int glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum_row_sharded(
    const glowb200_slws_job *jobs, int64_t num_jobs, int64_t max_segments, int kind,
    int indices_are_int64, int64_t in_line_size, int64_t out_line_size, void *workspace,
    size_t workspace_bytes, int32_t *status, glowb200_stream_t stream);

/* EmbeddingBagByteRowwiseOffsets (and its 4-bit form).
 * Replaces libjit_embedding_bag_byte_rowwise_offsets_f (libjit.cpp:2454-2481) and
 * fwdEmbeddingBagByteRowwiseOffsetsImpl (InterpreterNodes.cpp:5896-5986).  `offsets` has the
 * indices' integer type and `num_offsets` entries; bag i spans offsets[i]..offsets[i+1], the
 * last one ending at num_indices unless has_end_offset (then the last entry only closes the
 * previous bag).  dest has num_offsets - has_end_offset rows. */
int glowb200_embedding_bag_byte_rowwise_offsets(
    void *dest, const void *data, int kind, int64_t rows, const void *weights, const void *indices,
    const void *offsets, int indices_are_int64, int64_t num_offsets, int64_t num_indices,
    int64_t in_line_size, int64_t out_line_size, int has_end_offset, int out_is_fp16,
    int use_fp16_accumulation, void *workspace, size_t workspace_bytes, int32_t *status,
    glowb200_stream_t stream);

/* IntNBitSplitEmbeddingBags / IntNBitSplitEmbeddingWeightedBags: table-batched embedding bags.
 * Replaces fwdIntNBitSplitEmbeddingBagsInst / fwdIntNBitSplitEmbeddingWeightedBagsInst
 * (lib/Backends/Interpreter/InterpreterNodes.cpp:6593-6738, row helpers :42-114); the argument
 * list is the node's operand list (Function::createIntNBitSplitEmbeddingWeightedBags).
 *   dev_weights / uvm_weights   byte buffers holding the rows of all tables; table t reads
 *                               dev_weights when weights_placements[t] == 3 (HOST), uvm_weights
 *                               otherwise; placement 0 (DEVICE) is refused like in the reference
 *   weights_offsets [T]         byte offset of table t in its buffer (int32 or int64)
 *   weights_tys [T]             0 fp32, 1 fp16, 2 int8, 3 int4 (SplitEmbeddingSparseType,
 *                               include/glow/Graph/Nodes.h:302-309); int2 is refused
 *   dim_offsets [T+1]           table t has dim_offsets[t+1]-dim_offsets[t] columns and fills
 *                               columns dim_offsets[t].. of the result
 *   indices [num_indices], offsets [T*bags_per_table + 1]  same integer type; bag (t, b) is
 *                               offsets[t*B+b] .. offsets[t*B+b+1]
 *   pooling_mode                0 sum, 1 mean (bag length converted to the result type), 2 as 0
 *   indice_weights              NULL (unweighted node) or fp32 / fp16 [num_indices]
 *   dest                        [bags_per_table, total_dims] fp32 or fp16; sums are carried in
 *                               the result type (an fp16 result rounds after every row)
 *   scale_offset_is_fp32        int8 / int4 rows start with two fp32 instead of two fp16
 *                               (glow::flags::ConvertFusedScaleOffsetToFP32)
 *   row_alignment               rows are padded to this many bytes
 *                               (glow::interpreter::flags::RowAlignmentBytes, 16)
 * All table-description arrays are device pointers (they are operands of the node).  Rows that
 * reach outside their buffer raise GLOWB200_STATUS_INDEX_OUT_OF_RANGE and are skipped; results
 * are bit-identical to the Interpreter's. */
int glowb200_int_nbit_split_embedding_bags(
    void *dest, const void *dev_weights, int64_t dev_weights_bytes, const void *uvm_weights,
    int64_t uvm_weights_bytes, const int32_t *weights_placements, const void *weights_offsets,
    int weights_offsets_are_int64, const uint8_t *weights_tys, const int32_t *dim_offsets,
    int64_t num_tables, int64_t total_dims, const void *indices, const void *offsets,
    int indices_are_int64, int64_t num_indices, int64_t bags_per_table, int pooling_mode,
    const void *indice_weights, int indice_weights_are_fp16, int out_is_fp16,
    int scale_offset_is_fp32, int row_alignment, int32_t *status, glowb200_stream_t stream);

/* SparseLengthsWeightedSum / SparseLengthsSum over an fp32 table.
 * Replaces libjit_sparse_lengths_weighted_sum_f_u / _f_i32 and libjit_sparse_lengths_sum_f_u /
 * _f_i32 (lib/LLVMIRCodeGen/libjit/libjit.cpp:2318-2346, generic bodies :1164-1198).
 *   dest [segments, line_size] fp32; data [rows, line_size] fp32; weights fp32 [num_indices],
 *   or NULL for the unweighted sum (every row added as it is).
 * Each result element is accumulated in index order with separate multiply and add, so the
 * result is bit-identical to the reference kernel built without fast-math.
 * workspace: glowb200_slws_workspace_bytes(segments, 1). */
int glowb200_sparse_lengths_weighted_sum_f32(float *dest, const float *data, int64_t rows,
                                             const float *weights, const void *indices,
                                             int indices_are_int64, const int32_t *lengths,
                                             int64_t segments, int64_t num_indices,
                                             int64_t line_size, void *workspace,
                                             size_t workspace_bytes, int32_t *status,
                                             glowb200_stream_t stream);

/* RowwiseQuantizedSparseLengthsWeightedSum: uint8 table with per-row fp32 scale and offset in
 * separate vectors, value = scale[row] * q + offset[row].
 * Replaces libjit_rowwise_quantized_sparse_lengths_weighted_sum_f_u / _f_i32
 * (libjit.cpp:2400-2414, generic body :1232-1251).  Same ordering guarantee as above. */
int glowb200_rowwise_quantized_sparse_lengths_weighted_sum_f32(
    float *dest, const uint8_t *data, const float *scales, const float *offsets, int64_t rows,
    const float *weights, const void *indices, int indices_are_int64, const int32_t *lengths,
    int64_t segments, int64_t num_indices, int64_t line_size, void *workspace,
    size_t workspace_bytes, int32_t *status, glowb200_stream_t stream);

/* Weight preparation on the device (host weight preparation for weights already resident on the GPU).
 * glowb200_tensor_rowwise_quantize_i8_device: tensorRowwiseQuantization<float,int32_t,int8_t>
 * (include/glow/Quantization/Base/Base.h:522-576) -- every row of an fp32 [rows, cols] matrix gets
 * its own parameters from its min and max (schema as glowb200_choose_quantization_params) and is
 * quantized with them; same bytes as the host function glowb200_tensor_rowwise_quantize_i8.
 * glowb200_quantize_rows_i8_device: quantizeTensor with given per-row parameters
 * (lib/Quantization/Base/Base.cpp:760-777), the element pass of the channelwise filter
 * preparation once glowb200_channelwise_conv_prepare's parameter rules have run. */
int glowb200_tensor_rowwise_quantize_i8_device(const float *in, int64_t rows, int64_t cols,
                                               int schema, int8_t *out, float *scales,
                                               int32_t *offsets, glowb200_stream_t stream);
int glowb200_quantize_rows_i8_device(const float *in, int64_t rows, int64_t cols,
                                     const float *scales, const int32_t *offsets, int8_t *out,
                                     glowb200_stream_t stream);

/* tensorFusedRowwiseQuantization<T> (include/glow/Quantization/Base/Base.h:598-678): an fp32
 * [rows, cols] table into the fused-rowwise format of `kind`,
 * out_line_size = cols (+8 | +4) for the 8-bit kinds, cols/2 (+8 | +4) for the 4-bit kinds.
 * The first is a HOST function (host pointers); the _device form is the same arithmetic as a
 * kernel over device pointers, for tables that are produced or already resident on the GPU.
 * Both give the bytes the reference gives. */
int glowb200_fused_rowwise_quantize(const float *in, int64_t rows, int64_t cols, int kind,
                                    uint8_t *out, int64_t out_line_size);
int glowb200_fused_rowwise_quantize_device(const float *in, int64_t rows, int64_t cols, int kind,
                                           uint8_t *out, int64_t out_line_size,
                                           glowb200_stream_t stream);

/* Re-lays a fused-rowwise table [rows, in_line_size] out with rows of `padded_line_size` bytes:
 * the payload (in_line_size - tail_bytes bytes) first, zero padding, then the scale/offset pair
 * (tail_bytes = 8 for the fp32 kinds, 4 for the fp16 kinds) as the last bytes of the row.  The
 * gather-pool entry points accept such a table with in_line_size = padded_line_size and the
 * original out_line_size -- the reference kernel addresses a row the same way
 * (lib/LLVMIRCodeGen/libjit/libjit.cpp:1263-1270: scale/offset at the end of inLineSize bytes,
 * outLineSize columns from its start) -- and give bit-identical results.  Why: a 72-byte row at
 * an 8-byte aligned address straddles 64-byte DRAM atoms and, half of the time, a 128-byte
 * line; a row that fills one aligned 128-byte line is one access.  Costs HBM capacity, so it is
 * the loader's choice (src and dst are device pointers and must not overlap). */
int glowb200_fused_rows_pad(const uint8_t *src, int64_t rows, int64_t in_line_size,
                            int64_t tail_bytes, uint8_t *dst, int64_t padded_line_size,
                            glowb200_stream_t stream);

/* Sum of the fp32 partial results of a row-range sharded table (one slab per shard,
 * `partial_stride` floats apart, added in slab order) into dest [n], fp32 or fp16 -- the single
 * rounding to fp16 that keeps the sharded operator on fp32 accumulation.  No reference
 * counterpart: Glow does not split an embedding table by rows. */
int glowb200_sum_partials(const float *partials, int64_t num_partials, int64_t partial_stride,
                          int64_t n, void *dest, int dest_is_fp16, glowb200_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Int8 dense layers (tensor cores: tcgen05 kind::i8, int32 accumulation, Glow's integer
 * requantisation in the epilogue; results are bit-identical to the CPU backend's)
 * ------------------------------------------------------------------------------------- */

/* quantizeScaleOffset32To8 (lib/Quantization/Base/Base.cpp:234-359): the integer pre-shift,
 * post-shift and multiplier that stand in for a float rescale factor.  HOST function. */
void glowb200_quantize_scale_offset_32to8(float scale, int32_t *pre, int32_t *post,
                                          int32_t *integer_scale);

/* The six per-row (per-output-channel) integer arrays of RowwiseQuantizedFullyConnected and
 * ChannelwiseQuantizedConvolution, derived as lib/LLVMIRCodeGen/LLVMIRGen.cpp:2245-2251 and
 * :2726-2730 do: matMulScale = in_scale * row_scales[j]; bias from bias_scales[j] / matMulScale
 * (num_bias_scales is 1 for the FC's single bias scale, else n); output from
 * matMulScale / out_scale.  HOST function over host arrays of n entries. */
int glowb200_rowwise_requant_params(const float *row_scales, int64_t n, float in_scale,
                                    const float *bias_scales, int64_t num_bias_scales,
                                    float out_scale, int32_t *bias_pre, int32_t *bias_post,
                                    int32_t *bias_scale, int32_t *out_pre, int32_t *out_post,
                                    int32_t *out_scale_int);

/* chooseQuantizationParams without calibration (lib/Quantization/Base/Base.cpp:433-565): scale
 * and zero point for a float range.  schema: 0 Asymmetric, 1 Symmetric, 2 SymmetricWithUnsigned,
 * 3 SymmetricWithPower2Scale; quantized_bits 8, 16 or 32 (32 uses Glow's 30-bit range).  HOST. */
void glowb200_choose_quantization_params(float min, float max, int schema, int quantized_bits,
                                         float *scale, int32_t *offset);

/* tensorRowwiseQuantization<float,int32_t,int8_t> (include/glow/Quantization/Base/Base.h:522-576),
 * what Function::createRowwiseQuantizedFullyConnected (lib/Graph/Graph.cpp:1198-1246) runs on a
 * constant weight matrix at compile time.  HOST function over host arrays. */
int glowb200_tensor_rowwise_quantize_i8(const float *in, int64_t rows, int64_t cols, int schema,
                                        int8_t *out, float *scales, int32_t *offsets);

/* Bias to int32 with a given scale / offset (quantization::quantize, Base.h:322-329, clipped to
 * the 30-bit range of getQuantizedRange, Base.cpp:361-403).  HOST function. */
int glowb200_quantize_bias_i32(const float *in, int64_t n, float scale, int32_t offset, int32_t *out);

/* Constants of a ChannelwiseQuantizedConvolution from a float filter [out_channels, k] and a
 * float bias: what Function::createChannelwiseQuantizedConv (lib/Graph/Graph.cpp:3525-3700)
 * computes at graph-construction time -- per-channel filter scale/offset, int32 bias with
 * offset 0 and scale in_scale * filter_scale (specializeBiasWeightsQuantizationParams,
 * lib/Quantization/Base/Base.cpp:595-629), both tensors quantized.  HOST function. */
int glowb200_channelwise_conv_prepare(const float *filter, const float *bias, int64_t out_channels,
                                      int64_t k, float in_scale, int schema, int8_t *filter_q,
                                      float *filter_scales, int32_t *filter_offsets,
                                      int32_t *bias_q, float *bias_scales, int32_t *bias_offsets);

/* Hints in `flags`. */
#define GLOWB200_FC_WEIGHT_OFFSETS_ZERO 1      /* every weight offset is 0: skips the input row sums */
#define GLOWB200_FC_FORCE_ANY_SHAPE_KERNEL 2   /* run the plain one-thread-per-output kernel          */
#define GLOWB200_FC_FUSE_RELU 4                /* max(x, out_offset) in the epilogue: the int8 Relu that
                                                  follows the layer when both share one output type    */
#define GLOWB200_FC_BIAS_INT8 8                /* `bias` holds int8 values: the reference's _i8_i8 entry
                                                 points (libjit_matmul.cpp:409-422, :438-450;
                                                 libjit_conv.cpp:512-527, :547-562).  Same arithmetic. */

/* Every device-side wait of this library (the tensor-core kernels wait on mbarriers for TMA
 * loads, MMA completion and buffer hand-over) is bounded: after about a second it gives up, raises
 * GLOWB200_STATUS_WAIT_TIMEOUT in the status word, frees its tensor memory and returns, so the
 * context stays usable and the host decides (the runtime reports RUNTIME_DEVICE_NONRECOVERABLE).
 * This entry point runs that wait routine alone, on a barrier nothing ever completes, with a limit
 * of `limit_cycles` SM clocks: two warps wait, the first must run out, the second must notice and
 * leave; *waiters_that_gave_up (device int32, zeroed by the caller) counts them, the status word
 * gets the time-out bit.  No reference counterpart. */
int glowb200_wait_limit_selftest(int64_t limit_cycles, int32_t *status, int32_t *waiters_that_gave_up,
                                 glowb200_stream_t stream);

/* The int8 rate of the tensor pipe itself, for use as a roofline denominator: one CTA per SM
 * issues `mmas_per_sm` 128 x 256 x 32 int8 MMAs back to back on operand tiles resident in shared
 * memory (no loads, no epilogue) and waits, bounded, for the last.  *ops_per_launch (host, may be
 * NULL) receives the integer operations of one launch (2 per multiply-add); the caller times the
 * launch with events.  The reference defines the metric, not a ceiling
 * (tests/benchmark/Int8GemmBench.h:222-224); no reference counterpart. */
int glowb200_i8_mma_issue_probe(int64_t mmas_per_sm, int64_t *ops_per_launch, int32_t *status,
                                glowb200_stream_t stream);

/* Scratch bytes the three entry points below may need for an [M,K] x [N,K]^T problem. */
size_t glowb200_i8_gemm_workspace_bytes(int64_t M, int64_t K, int64_t N);

/* sums[r] = sum_k matrix[r,k] (int8 [rows,K] -> int32 [rows]).  Lets a caller compute the row
 * sums of constant weights once, at network-load time, and pass them as `weights_row_sums`. */
int glowb200_i8_row_sums(const int8_t *matrix, int64_t rows, int64_t K, int32_t *sums,
                         glowb200_stream_t stream);

/* RowwiseQuantizedFullyConnected, int8 with int32 bias.
 * Replaces libjit_rowwise_quantized_fc_i8_i32 (lib/LLVMIRCodeGen/libjit/libjit_matmul.cpp:425-436,
 * body :284-316).  in [M,K]; weights [N,K] (not transposed: out = in * weights^T); bias,
 * weights_offsets and the six per-row requantisation arrays have N entries and are derived by
 * the caller exactly as lib/LLVMIRCodeGen/LLVMIRGen.cpp:2222-2320 derives them.
 * weights_row_sums: optional int32 [N] from glowb200_i8_row_sums (NULL: computed per call).
 * Environment: GLOWB200_GEMM_PAIR=1 (240-column tiles) or 2 (256-column tiles) makes products of
 * 256 rows or more, of this and the two entry points below, run on pairs of CTAs (one MMA over two
 * SMs, tcgen05 cta_group::2) -- same results; the default is one CTA per tile, which measured faster. */
int glowb200_rowwise_quantized_fc_i8_i32(
    int8_t *out, const int8_t *in, const int8_t *weights, const int32_t *bias,
    const int32_t *weights_offsets, const int32_t *bias_pre, const int32_t *bias_post,
    const int32_t *bias_scale, const int32_t *out_pre, const int32_t *out_post,
    const int32_t *out_scale, int64_t M, int64_t K, int64_t N, int32_t out_offset,
    int32_t in_offset, int32_t bias_offset, const int32_t *weights_row_sums, int flags,
    void *workspace, size_t workspace_bytes, int32_t *status, glowb200_stream_t stream);

/* FullyConnected, int8 with int32 bias, one quantisation per tensor.
 * Replaces libjit_fc_i8_i32 (libjit_matmul.cpp:395-407, body :254-280; scalars derived at
 * LLVMIRGen.cpp:2161-2220).  in [M,K]; weights [K,N].  weights_transposed: optional [N,K] copy
 * of the weights (a constant can be transposed once at load time); NULL: transposed per call
 * into the workspace. */
int glowb200_fc_i8_i32(int8_t *out, const int8_t *in, const int8_t *weights, const int32_t *bias,
                       int64_t M, int64_t K, int64_t N, int32_t out_offset, int32_t in_offset,
                       int32_t weights_offset, int32_t bias_offset, int32_t bias_pre,
                       int32_t bias_post, int32_t bias_scale, int32_t out_pre, int32_t out_post,
                       int32_t out_scale, const int8_t *weights_transposed, int flags,
                       void *workspace, size_t workspace_bytes, int32_t *status,
                       glowb200_stream_t stream);

/* QuantizationProfile: running min / max and histogram of a tensor on the device.
 * Replaces libjit_quantization_profile (lib/LLVMIRCodeGen/libjit/libjit.cpp:3440-3523; the same
 * algorithm as generateTensorHistogram, lib/Quantization/Base/Profile.cpp:36-112).  comp_info
 * (device, 2 floats) holds the running {min, max}, initialised by the caller to {FLT_MAX,
 * -FLT_MAX}; histogram (device, `bins` floats) the running counters.  When the range grows the
 * existing bins are redistributed as the reference does; results are bit-identical to libjit
 * built without fast-math. */
size_t glowb200_quantization_profile_workspace_bytes(int64_t bins);
int glowb200_quantization_profile(const float *input, int64_t size, float *comp_info,
                                  float *histogram, int64_t bins, void *workspace,
                                  size_t workspace_bytes, glowb200_stream_t stream);

/* DynamicRowwiseQuantizedFullyConnected / DynamicQuantizedFullyConnected.
 * Replace fwdDynamicRowwiseQuantizedFullyConnectedInst and fwdDynamicQuantizedFullyConnectedInst
 * (lib/Backends/Interpreter/InterpreterNodes.cpp:4677-4790; symmetric, per batch element -- the
 * only mode the reference implements).  in [M,K] fp16; weights [K,N] int8 as the node holds
 * them (weights_transposed: the [N,K] form, e.g. transposed once at load time; either may be
 * NULL); bias [N] fp32; scales [N] fp32 and offsets [N] int32 per output column (the rowwise
 * node) or one weights_scale / weights_offset (the per-tensor node); out [M,N] fp16.
 * Every input row is quantized to int8 with its own Symmetric parameters, the int32 sums come
 * from the tensor cores, and out = fp16(float(sum) * (row scale * scales[j]) + bias[j]) with the
 * reference's roundings: results are bit-identical to the Interpreter's.
 * flags: GLOWB200_FC_WEIGHT_OFFSETS_ZERO, GLOWB200_FC_FORCE_ANY_SHAPE_KERNEL.  The workspace
 * (256-byte aligned) must hold glowb200_dynamic_fc_workspace_bytes(M, K, N). */
size_t glowb200_dynamic_fc_workspace_bytes(int64_t M, int64_t K, int64_t N);
int glowb200_dynamic_rowwise_quantized_fc(void *out, const void *in, const int8_t *weights,
                                          const float *bias, const float *scales,
                                          const int32_t *offsets, int64_t M, int64_t K, int64_t N,
                                          const int8_t *weights_transposed, int flags,
                                          void *workspace, size_t workspace_bytes, int32_t *status,
                                          glowb200_stream_t stream);
int glowb200_dynamic_quantized_fc(void *out, const void *in, const int8_t *weights,
                                  const float *bias, float weights_scale, int32_t weights_offset,
                                  int64_t M, int64_t K, int64_t N, const int8_t *weights_transposed,
                                  int flags, void *workspace, size_t workspace_bytes,
                                  int32_t *status, glowb200_stream_t stream);

/* MatMul, int8.  Replaces libjit_matmul_i8 (libjit_matmul.cpp:353-371; scalars derived at
 * LLVMIRGen.cpp:2098-2137).  lhs [M,K], rhs [K,N]. */
int glowb200_matmul_i8(int8_t *out, const int8_t *lhs, const int8_t *rhs, int64_t M, int64_t K,
                       int64_t N, int32_t out_offset, int32_t lhs_offset, int32_t rhs_offset,
                       int32_t out_pre, int32_t out_post, int32_t out_scale, int flags,
                       void *workspace, size_t workspace_bytes, int32_t *status,
                       glowb200_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Int8 convolution (NHWC activations, filter [outC, kH, kW, inC/group]).  The four-entry shape
 * arrays are HOST arrays, laid out as the reference passes them: dims {N,H,W,C}, kernels {h,w},
 * strides {h,w}, pads {top,left,bottom,right} (only top and left are read, like the reference),
 * dilation {h,w}.  act_type / act_args follow glow::FusedActivation as libjit_activation_i32
 * reads them (0 none, 1 relu, 2 clip {min,max}, 5 leaky relu {pre,post,scale}); act_args is a
 * HOST array.
 * ------------------------------------------------------------------------------------- */
size_t glowb200_conv2d_workspace_bytes(const int64_t *out_dims, const int64_t *in_dims,
                                       const int64_t *filter_dims, const int64_t *kernels,
                                       const int64_t *strides, const int64_t *pads, int64_t group,
                                       const int64_t *dilation);

/* ChannelwiseQuantizedConvolution (2-D), int8 with int32 bias.
 * Replaces libjit_channelwise_quantized_conv2d_i8_i32 (lib/LLVMIRCodeGen/libjit/libjit_conv.cpp:
 * 530-545, body :151-239; per-channel integers derived at LLVMIRGen.cpp:2695-2798).
 * filter_row_sums: optional int32 [outC] = glowb200_i8_row_sums(filter as [outC, kH*kW*inC]);
 * flags: GLOWB200_FC_WEIGHT_OFFSETS_ZERO when every filter offset is 0 (symmetric filters). */
int glowb200_channelwise_quantized_conv2d_i8_i32(
    int8_t *out, const int8_t *in, const int8_t *filter, const int32_t *bias,
    const int64_t *out_dims, const int64_t *in_dims, const int64_t *filter_dims,
    const int64_t *kernels, const int64_t *strides, const int64_t *pads, int64_t group,
    const int64_t *dilation, int32_t out_offset, int32_t in_offset,
    const int32_t *filter_offsets, const int32_t *bias_offsets, const int32_t *bias_pre,
    const int32_t *bias_post, const int32_t *bias_scale, const int32_t *out_pre,
    const int32_t *out_post, const int32_t *out_scale, int32_t act_type, const int32_t *act_args,
    const int32_t *filter_row_sums, int flags, void *workspace, size_t workspace_bytes,
    int32_t *status, glowb200_stream_t stream);

/* Convolution (2-D), int8 with int32 bias, one quantisation per tensor.
 * Replaces libjit_conv2d_i8_i32 (libjit_conv.cpp:496-510, body :49-147; scalars derived at
 * LLVMIRGen.cpp:2501-2599).  The reference's depthUnroll argument only blocks its loops and
 * has no counterpart here. */
int glowb200_conv2d_i8_i32(
    int8_t *out, const int8_t *in, const int8_t *filter, const int32_t *bias,
    const int64_t *out_dims, const int64_t *in_dims, const int64_t *filter_dims,
    const int64_t *kernels, const int64_t *strides, const int64_t *pads, int64_t group,
    int32_t out_offset, int32_t in_offset, int32_t filter_offset, int32_t bias_offset,
    int32_t bias_pre, int32_t bias_post, int32_t bias_scale, int32_t out_pre, int32_t out_post,
    int32_t out_scale, const int64_t *dilation, int32_t act_type, const int32_t *act_args,
    int flags, void *workspace, size_t workspace_bytes, int32_t *status, glowb200_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Int8 glue operators (n = element count; tensors are dense)
 * ------------------------------------------------------------------------------------- */

/* ElementAdd int8: libjit_element_add_kernel_i8 (libjit.cpp:1593-1603); the two triples come
 * from lhsScale/destScale and rhsScale/destScale (LLVMIRGen.cpp:1716-1771). */
int glowb200_element_add_i8(int8_t *dest, const int8_t *lhs, const int8_t *rhs, int64_t n,
                            int32_t dest_offset, int32_t lhs_offset, int32_t rhs_offset,
                            int32_t lhs_pre, int32_t lhs_post, int32_t lhs_scale, int32_t rhs_pre,
                            int32_t rhs_post, int32_t rhs_scale, glowb200_stream_t stream);
/* ElementAdd / Sub / Max / Min int8: the arithmetic mini-kernels libjit_element_{add,sub,max,min}_kernel_i8
 * (DEFINE_DATA_PARALLEL_KERNEL_QUANTIZED, libjit.cpp:1593-1603, 1675-1682; triples derived at
 * LLVMIRGen.cpp:1716-1776 from lhsScale / destScale and rhsScale / destScale). */
#define GLOWB200_BINARY_ADD 0
#define GLOWB200_BINARY_SUB 1
#define GLOWB200_BINARY_MAX 2
#define GLOWB200_BINARY_MIN 3
int glowb200_element_binary_i8(int op, int8_t *dest, const int8_t *lhs, const int8_t *rhs, int64_t n,
                               int32_t dest_offset, int32_t lhs_offset, int32_t rhs_offset,
                               int32_t lhs_pre, int32_t lhs_post, int32_t lhs_scale, int32_t rhs_pre,
                               int32_t rhs_post, int32_t rhs_scale, glowb200_stream_t stream);

/* ElementMul / ElementDiv int8: libjit_element_mul_kernel_i8 / libjit_element_div_kernel_i8
 * (DEFINE_DATA_PARALLEL_KERNEL_QUANTIZED_M, libjit.cpp:1610-1619, 1683-1684); one triple, from
 * lhsScale * rhsScale / destScale (mul) or lhsScale / (rhsScale * destScale) (div),
 * LLVMIRGen.cpp:1927-2035.  A zero divisor yields the result offset. */
int glowb200_element_muldiv_i8(int is_div, int8_t *dest, const int8_t *lhs, const int8_t *rhs,
                               int64_t n, int32_t dest_offset, int32_t lhs_offset,
                               int32_t rhs_offset, int32_t pre, int32_t post, int32_t scale,
                               glowb200_stream_t stream);

/* BatchedAdd int8: libjit_batchedadd_i8 and, with an int32 slice, libjit_batchedadd_i32_i8
 * (libjit.cpp:997-1015, 1945-1969).  batch / dest [num_slices, slice_size], slice [slice_size]. */
int glowb200_batched_add_i8(int8_t *dest, const int8_t *batch, const void *slice, int slice_is_int32,
                            int64_t num_slices, int64_t slice_size, int32_t dest_offset,
                            int32_t batch_offset, int32_t slice_offset, int32_t batch_pre,
                            int32_t batch_post, int32_t batch_scale, int32_t slice_pre,
                            int32_t slice_post, int32_t slice_scale, glowb200_stream_t stream);

/* Add followed by the int8 Relu of a residual block -- glowb200_element_add_i8 then
 * glowb200_element_maxsplat_i8(splat) on its result -- in one pass over memory (the pair is two
 * instructions in Glow's IR: ElementAdd, then the CPU backend's CPUMaxSplat,
 * lib/Backends/CPU/Transforms.cpp:83-113).  Bit-identical to the two calls. */
int glowb200_element_add_maxsplat_i8(int8_t *dest, const int8_t *lhs, const int8_t *rhs, int64_t n,
                                     int32_t dest_offset, int32_t lhs_offset, int32_t rhs_offset,
                                     int32_t lhs_pre, int32_t lhs_post, int32_t lhs_scale,
                                     int32_t rhs_pre, int32_t rhs_post, int32_t rhs_scale,
                                     int32_t splat, glowb200_stream_t stream);

/* Relu int8: libjit_element_relu_i8 (libjit.cpp:1850-1858). */
int glowb200_element_relu_i8(int8_t *dest, const int8_t *src, int64_t n, int32_t src_offset,
                             int32_t dest_offset, int32_t dest_pre, int32_t dest_post,
                             int32_t dest_scale, glowb200_stream_t stream);
/* max(x, constant): libjit_element_maxsplat_kernel_i8 (lib/Backends/CPU/libjit_cpu/libjit_cpu.cpp:
 * 39-44), what the CPU backend turns a quantized Relu into (lib/Backends/CPU/Transforms.cpp:83-113). */
int glowb200_element_maxsplat_i8(int8_t *dest, const int8_t *src, int64_t n, int32_t splat,
                                 glowb200_stream_t stream);
/* Splat: every element of dest [n] set to `value`, as fp32 or (dest_is_fp16) rounded to fp16
 * (libjit_splat_kernel_f, libjit.cpp; the ones that weight a lowered SparseLengthsSum,
 * lib/Optimizer/Lower/Lower.cpp:1590-1606). */
int glowb200_splat_f(void *dest, int64_t n, float value, int dest_is_fp16, glowb200_stream_t stream);
/* RescaleQuantized int8: libjit_element_rescale_kernel_i8 (libjit.cpp:3030-3038). */
int glowb200_element_rescale_i8(int8_t *dest, const int8_t *src, int64_t n, int32_t out_offset,
                                int32_t in_offset, int32_t pre, int32_t post, int32_t scale,
                                glowb200_stream_t stream);
/* Quantize fp32 -> int8: libjit_element_quantize_kernel_i8 (libjit.cpp:2997-3002). */
int glowb200_element_quantize_i8(int8_t *dest, const float *src, int64_t n, float scale,
                                 int32_t offset, glowb200_stream_t stream);
/* Dequantize int8 -> fp32: libjit_element_dequantize_kernel_i8 (libjit.cpp:3014-3018). */
int glowb200_element_dequantize_i8(float *dest, const int8_t *src, int64_t n, float scale,
                                   int32_t offset, glowb200_stream_t stream);
/* MaxPool int8, NHWC: libjit_max_pool_i8 (libjit.cpp:2592-2597, body :811-870). */
int glowb200_max_pool_i8(const int8_t *in, int8_t *out, const int64_t *in_dims,
                         const int64_t *out_dims, const int64_t *kernels, const int64_t *strides,
                         const int64_t *pads, int32_t out_offset, glowb200_stream_t stream);
/* AvgPool int8, NHWC: libjit_avg_pool_i8 (libjit.cpp:2812-2897). */
int glowb200_avg_pool_i8(const int8_t *in, int8_t *out, const int64_t *in_dims,
                         const int64_t *out_dims, const int64_t *kernels, const int64_t *strides,
                         const int64_t *pads, int count_include_pads, int32_t out_offset,
                         int32_t in_offset, int32_t out_pre, int32_t out_post, int32_t out_scale,
                         glowb200_stream_t stream);
/* Transpose of a tensor of up to 4 dimensions with 1- or 4-byte elements (libjit_transpose_i8 /
 * _f, libjit.cpp:1945-...): dest dims[i] = src_dims[shuffle[i]].  src_dims / shuffle are HOST arrays. */
int glowb200_transpose(const void *src, void *dest, const int64_t *src_dims, const int32_t *shuffle,
                       int num_dims, int element_bytes, glowb200_stream_t stream);
/* Quantize fp32 -> int8 and Transpose in one pass: dest = transpose(quantize(src)), the pair Glow's
 * optimizer leaves when it sinks a Transpose below the Quantize that consumes it
 * (lib/Optimizer/GraphOptimizer/GraphOptimizer.cpp:1076-1086) -- an NCHW float input becoming the
 * NHWC int8 input of the first convolution.  Element for element the result of
 * glowb200_element_quantize_i8 (libjit.cpp:2997-3002) followed by glowb200_transpose. */
int glowb200_quantize_transpose_i8(int8_t *dest, const float *src, const int64_t *src_dims,
                                   const int32_t *shuffle, int num_dims, float scale, int32_t offset,
                                   glowb200_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Recommendation-model pieces
 * ------------------------------------------------------------------------------------- */

/* Pairwise-dot feature interaction.  For each of `batch` samples: n = tables + 1 vectors of `dim`
 * fp32 values (v_0 = dense[b], v_t = pooled[b, t-1]); the result row is v_0 followed by the
 * dot products v_i.v_j for j < i in row-major order (dim + n(n-1)/2 values), written as fp32
 * (out_f32) or quantized to int8 with quant_scale / quant_offset (out_i8) -- exactly one of the
 * two outputs is given.  ld_* are row pitches in elements.  The reference composes this from
 * Concat / Reshape / BatchMatMul / flatten nodes
 * (tests/unittests/RecommendationSystemTest.cpp:640-680) and has no single kernel for it. */
int glowb200_pairwise_dot_interaction(const float *dense, int64_t ld_dense, const float *pooled,
                                      int64_t ld_pooled, int64_t batch, int64_t tables, int64_t dim,
                                      float *out_f32, int8_t *out_i8, int64_t ld_out,
                                      float quant_scale, int32_t quant_offset,
                                      glowb200_stream_t stream);

/* Device buffers other GPUs of the node can store into (one process per GPU): create exports
 * a 64-byte handle, open maps a peer's handle, close / destroy undo them.  Set-up time only:
 * create and destroy allocate and free device memory.  The reference hands tensors between
 * devices through host buffers (lib/Runtime/Executor/NetworkExecutionState.cpp:191-203); this
 * replaces that hand-off for the pooled embeddings. */
int glowb200_peer_buffer_create(size_t bytes, void **device_ptr, void *ipc_handle_64_bytes);
int glowb200_peer_buffer_open(const void *ipc_handle_64_bytes, void **device_ptr);
int glowb200_peer_buffer_close(void *device_ptr);
int glowb200_peer_buffer_destroy(void *device_ptr);
/* Rendezvous of the ranks that store into each other's peer buffers, as one small kernel on
 * the stream (no collective library call, replayable from a CUDA graph): `my_flags` is this
 * rank's flag buffer -- a peer buffer of 8 * (world + 1) bytes, zeroed once -- and
 * `peer_flags_device_array` a DEVICE array of the `world` ranks' flag-buffer addresses as this
 * rank has them mapped (its own at index `rank`).  The kernel tells every peer that the work
 * queued before it on the stream is stored, then waits until every peer has said the same for
 * the same step; what is queued behind it may read what the peers stored.  The wait gives up
 * after `limit_cycles` SM clocks and raises GLOWB200_STATUS_WAIT_TIMEOUT.  Replaces the
 * host-mediated hand-off between the partitions of a network
 * (lib/Runtime/Executor/NetworkExecutionState.cpp:129-255); no kernel counterpart in the reference. */
int glowb200_peer_rendezvous(void *my_flags, void *const *peer_flags_device_array, int world, int rank,
                             int64_t limit_cycles, int32_t *status, glowb200_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Host runtime: the compiled-function and device-manager layer of a Glow backend, written
 * against this library (runtime.cu).  A function is a symbol table over three slabs
 * (constants, placeholders, activations: glow::RuntimeBundle, include/glow/Backend/
 * BackendUtils.h:66-170) plus a flat instruction list; glowb200_function_compile derives the
 * integer requantisation parameters from the float scales the way LLVMIRGen does and lays the
 * slabs out.  The device manager mirrors glow::DeviceManager (include/glow/Backends/
 * DeviceManager.h:47-241) as CPUDeviceManager implements it
 * (lib/Backends/CPU/CPUDeviceManager.cpp:65-179).  Calls are synchronous unless they say
 * otherwise; a Glow QueueBackedDeviceManager would make them from its one worker thread.
 * Operand and attribute layouts of every instruction kind are listed above
 * glowb200_function_compile in runtime.cu.
 * ------------------------------------------------------------------------------------- */
#define GLOWB200_SYMBOL_CONSTANT 0
#define GLOWB200_SYMBOL_PLACEHOLDER 1
#define GLOWB200_SYMBOL_ACTIVATION 2
/* A placeholder that is written once and stays put (Placeholder::isStatic, include/glow/Graph/
 * Nodes.h; the embedding tables of a recommendation model): lives beside the constants, shared
 * by all execution contexts, filled by glowb200_device_manager_transfer_static_placeholder. */
#define GLOWB200_SYMBOL_STATIC 3

#define GLOWB200_INSTR_FRWQ_SLWS 1
#define GLOWB200_INSTR_RWQ_FC 2
#define GLOWB200_INSTR_CWQ_CONV 3
#define GLOWB200_INSTR_ADD 4
#define GLOWB200_INSTR_MAXSPLAT 5
#define GLOWB200_INSTR_QUANTIZE 6
#define GLOWB200_INSTR_DEQUANTIZE 7
#define GLOWB200_INSTR_MAXPOOL 8
#define GLOWB200_INSTR_AVGPOOL 9
#define GLOWB200_INSTR_TRANSPOSE 10
#define GLOWB200_INSTR_COPY 11
#define GLOWB200_INSTR_ADD_MAXSPLAT 12   /* ElementAdd followed by the max-with-immediate of a Relu */
#define GLOWB200_INSTR_RELU 13
#define GLOWB200_INSTR_RESCALE 14
#define GLOWB200_INSTR_FC_I8 15          /* FullyConnected, per-tensor quantized */
#define GLOWB200_INSTR_MATMUL_I8 16
#define GLOWB200_INSTR_SPLAT 17          /* fp32 / fp16 fill (the weights of a lowered SparseLengthsSum) */
#define GLOWB200_INSTR_INSERT_TENSOR 18  /* a [rows, width] block into a wider tensor (lowered Concat) */
#define GLOWB200_INSTR_PAIRWISE_DOT 19
#define GLOWB200_INSTR_SLWS_F32 20       /* SparseLengths(Weighted)Sum over an fp32 table */
#define GLOWB200_INSTR_RWQ_SLWS 21       /* RowwiseQuantizedSparseLengthsWeightedSum */
#define GLOWB200_INSTR_EMBEDDING_BAG 22  /* EmbeddingBagByteRowwiseOffsets */
#define GLOWB200_INSTR_SPLIT_EMBEDDING 23 /* IntNBitSplitEmbedding(Weighted)Bags */
#define GLOWB200_INSTR_DYN_QUANTIZED_FC 24 /* Dynamic(Rowwise)QuantizedFullyConnected */
#define GLOWB200_INSTR_BINARY_I8 25       /* ElementSub / Max / Min (and Add) */
#define GLOWB200_INSTR_MULDIV_I8 26       /* ElementMul / ElementDiv */
#define GLOWB200_INSTR_BATCHED_ADD_I8 27  /* BatchedAdd, int8 or int32 slice */

typedef struct glowb200_function glowb200_function;
typedef struct glowb200_device_manager glowb200_device_manager;

glowb200_function *glowb200_function_create(const char *name);
void glowb200_function_destroy(glowb200_function *f);
/* Returns the symbol id (>= 0) or -1.  Constants carry their host data (copied). */
int glowb200_function_add_symbol(glowb200_function *f, const char *name, int kind, size_t bytes,
                                 const void *host_data);
int glowb200_function_add_instruction(glowb200_function *f, int kind, const int32_t *operands,
                                      int num_operands, const int64_t *int_attrs, int num_int_attrs,
                                      const float *float_attrs, int num_float_attrs);
/* The same with a byte offset per operand: operand i is the part of its symbol that starts
 * operand_byte_offsets[i] bytes in -- a TensorView of a larger tensor (include/glow/IR/Instrs.h,
 * TensorViewInst with its offsets).  compile checks offset + size against the symbol. */
int glowb200_function_add_instruction_views(glowb200_function *f, int kind, const int32_t *operands,
                                            const int64_t *operand_byte_offsets, int num_operands,
                                            const int64_t *int_attrs, int num_int_attrs,
                                            const float *float_attrs, int num_float_attrs);
/* Besides laying out the slabs and deriving the integer parameters, compile turns every run of
 * consecutive, mutually independent FusedRowwiseQuantizedSparseLengthsWeightedSum instructions
 * over tables of one kind and row width into ONE batched launch (the per-table SparseLengthsSum
 * nodes of a recommendation model); results are bit-identical to the single launches. */
int glowb200_function_compile(glowb200_function *f);
size_t glowb200_function_constant_bytes(const glowb200_function *f);
/* How many batched pooling launches compile formed (0 before compile). */
int glowb200_function_batched_pooling_launches(const glowb200_function *f);
/* How many Quantize + Transpose pairs compile turned into one kernel each: a Quantize into an
 * activation that only the Transpose right behind it reads (0 before compile).  Same results. */
int glowb200_function_fused_quantize_transposes(const glowb200_function *f);

/* max_memory_bytes 0 = the device's free memory at init. */
glowb200_device_manager *glowb200_device_manager_create(int device_id, uint64_t max_memory_bytes);
int glowb200_device_manager_init(glowb200_device_manager *dm);
int glowb200_device_manager_add_network(glowb200_device_manager *dm, glowb200_function *f);
int glowb200_device_manager_evict_network(glowb200_device_manager *dm, const char *name);
/* Execution contexts networks are loaded with from now on (Backend::getContextCount,
 * include/glow/Backend/Backend.h:272-276): each has its own placeholders and activations
 * (constants and static placeholders are shared), so requests can overlap.  1 by default. */
int glowb200_device_manager_set_context_count(glowb200_device_manager *dm, int contexts);
/* Placeholder names paired with HOST buffers; every bound buffer is copied in before and out
 * after the run; a buffer shorter than its placeholder is a partial tensor (rest zeroed).
 * The _io form takes a direction per binding (GLOWB200_BINDING_INPUT: copied in only, _OUTPUT: copied
 * out only, both bits: both ways; directions NULL = both for all) -- the input / output marks of
 * Glow's symbol table (include/glow/Backend/BackendUtils.h:38-60). */
#define GLOWB200_BINDING_INPUT 1
#define GLOWB200_BINDING_OUTPUT 2
int glowb200_device_manager_run_function_io(glowb200_device_manager *dm, const char *name,
                                            const char *const *placeholder_names,
                                            void *const *host_buffers, const size_t *buffer_bytes,
                                            const int *directions, int num_bindings);
/* The asynchronous form of _run_function_io (DeviceManager::runFunction returns at once and
 * calls back, include/glow/Backends/DeviceManager.h:120-135; CPUDeviceManager.cpp:141-179 is the
 * synchronous body behind it): inputs go in on one stream, the kernels run on a second, results
 * leave on a third, ordered by events.  With two or more contexts the copies of neighbouring
 * requests overlap the kernels.  *ticket identifies the request; _wait blocks until its outputs
 * are in the host buffers and returns its result (what _run_function_io would have returned).
 * The host buffers must stay valid until then and should be pinned (_allocate_io_buffer:
 * DeviceManager::allocateDeviceIOBuffer, DeviceManager.h:150-160). */
int glowb200_device_manager_run_function_async(glowb200_device_manager *dm, const char *name,
                                               const char *const *placeholder_names,
                                               void *const *host_buffers, const size_t *buffer_bytes,
                                               const int *directions, int num_bindings,
                                               int64_t *ticket);
int glowb200_device_manager_wait(glowb200_device_manager *dm, int64_t ticket);
void *glowb200_device_manager_allocate_io_buffer(glowb200_device_manager *dm, size_t bytes);
void glowb200_device_manager_free_io_buffer(glowb200_device_manager *dm, void *buffer);
/* Device-resident tensors and static placeholders (DeviceManager::transferToDevice /
 * transferFromDevice / transferStaticPlaceholderToDevice, include/glow/Backends/DeviceManager.h:
 * 163-231, and the peer-to-peer hand-off between the partitions of a network): the device address
 * of a placeholder of a loaded network -- what is written there (by a copy, by another kernel, by a
 * peer GPU) is what the next run reads, and results can be read from there; _transfer_static_placeholder
 * copies a host buffer there once (embedding tables marked static); _run_function_resident runs the
 * network on the placeholders as they are, with no copies. */
int glowb200_device_manager_placeholder_address(glowb200_device_manager *dm, const char *name,
                                                const char *placeholder, void **device_ptr,
                                                size_t *bytes);
int glowb200_device_manager_transfer_static_placeholder(glowb200_device_manager *dm,
                                                        const char *name, const char *placeholder,
                                                        const void *host, size_t bytes);
int glowb200_device_manager_run_function_resident(glowb200_device_manager *dm, const char *name);
int glowb200_device_manager_run_function(glowb200_device_manager *dm, const char *name,
                                         const char *const *placeholder_names,
                                         void *const *host_buffers, const size_t *buffer_bytes,
                                         int num_bindings);
uint64_t glowb200_device_manager_maximum_memory(glowb200_device_manager *dm);
uint64_t glowb200_device_manager_available_memory(glowb200_device_manager *dm);
int glowb200_device_manager_is_memory_available(glowb200_device_manager *dm, uint64_t estimate);
int glowb200_device_manager_stop(glowb200_device_manager *dm);
void glowb200_device_manager_destroy(glowb200_device_manager *dm);

/* FusedRowwiseQuantizedSparseLengthsWeightedSum for callers that can neither allocate device
 * memory nor size a workspace per request.  (No counterpart in the reference: its CPU kernels
 * need no scratch.)  Think of a DeviceManager's request thread after every byte of HBM was
 * budgeted at network-load time -- a cudaMalloc there can fail against the budget and blocks
 * all streams of the device while it runs -- or of a plug-in that only ever receives buffers
 * from its host.  Same arguments and results as
 * glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum minus the workspace pair: the bag
 * boundaries go into an array built into the library (about 0.5 MB of device memory on every
 * GPU that loads it, held until the process exits).
 *   - At most glowb200_slws_static_scratch_max_segments() (65536) bags per call; more is
 *     refused with GLOWB200_ERR_UNSUPPORTED and a message, nothing is launched.
 *   - The first call on each device looks the array's device address up (with that device
 *     current).  Make that first call during set-up, before any stream capture is begun.
 *   - All calls on a device share the one array.  Calls on the same stream are ordered and
 *     safe; calls that can overlap on the GPU (different streams, different host threads on
 *     different streams) race on it and must be serialised by the caller.
 *   - This entry point calls no cudaMalloc / cudaFree or any other allocating routine.  What it
 *     cannot rule out is the CUDA runtime's own lazy module loading: the first launch of each
 *     kernel variant (table kind x index type x row width class) may load its code then, and the
 *     set-up call warms only the variant it uses -- make one set-up call per shape that will be
 *     served, or run with CUDA_MODULE_LOADING=EAGER.
 *   - The looked-up address is kept per device ordinal for the life of the process; it does not
 *     survive a cudaDeviceReset (a process that resets a device must not call this afterwards). */
int64_t glowb200_slws_static_scratch_max_segments(void);
int glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum_static_scratch(
    void *dest, const void *data, int kind, int64_t rows, const void *weights, const void *indices,
    int indices_are_int64, const int32_t *lengths, int64_t segments, int64_t num_indices,
    int64_t in_line_size, int64_t out_line_size, int out_is_fp16, int use_fp16_accumulation,
    int32_t *status, glowb200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* GLOW_B200_H */
