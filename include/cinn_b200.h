/*
 * C ABI of the B200 fused-group kernel library (libcinn_b200.so).
 *
 * The library is a drop-in for one path of CINN: the kernels it generates at run time for HLIR fused op
 * groups (elementwise / broadcast / reduction), the host stubs that launch them, and the launch primitive.
 * Everything crosses this boundary as plain pointers and sizes; the argument structures are the
 * reference's own (see cinn_runtime_abi.h).  No function here throws; functions returning int give 0 on
 * success and a negative CINN_B200_E* code otherwise, with a message available from cinn_b200_last_error().
 *
 * Each declaration names the reference interface it replaces (paths are inside the CINN project).
 */
#ifndef CINN_B200_H_
#define CINN_B200_H_

#include "cinn_runtime_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

#define CINN_B200_OK 0
#define CINN_B200_EINVAL (-1)     /* malformed argument (null pointer, wrong count, wrong type tag) */
#define CINN_B200_ENOMATCH (-2)   /* no prebuilt kernel covers the group (there is no fallback) */
#define CINN_B200_ENOTFOUND (-3)  /* unknown function or kernel name */
#define CINN_B200_ECUDA (-4)      /* a CUDA runtime call failed */
#define CINN_B200_ESHAPE (-5)     /* a buffer's type or element count differs from the compiled group's */
#define CINN_B200_ENOSPACE (-6)   /* table full / caller buffer too small */

/* Message of the most recent failure on the calling thread ("" if none).  The pointer stays valid until the
 * next failing call on the same thread.  Replaces the reference's LOG(FATAL)/abort convention
 * (cinn/backends/cuda_util.h:30-45) with a status + message. */
const char* cinn_b200_last_error(void);

/* ---- launch primitive ----------------------------------------------------------------------------- */

/*
 * Same name, signature and argument unpacking as cinn/runtime/cuda/cuda_util.h:75-84 (implementation
 * cinn/runtime/cuda/cuda_util.cc:78-118): v_args is a cinn_pod_value_t[num_args]; a buffer argument
 * contributes the address of its `memory` field as the kernel parameter, any other argument the address
 * of its 8-byte payload.  kernel_fn is a handle from cinn_b200_get_kernel() (the reference passes a
 * CUfunction published as "<fn>_kernel_ptr_", cinn/backends/compiler.cc:133-140).  Dynamic shared memory
 * is 0 as in the reference.  Failures are reported through cinn_b200_last_error() and, when the
 * environment variable CINN_B200_ABORT_ON_ERROR is set, abort() like the reference does.
 */
void cinn_call_cuda_kernel(void* kernel_fn, void* v_args, int num_args, int grid_x, int grid_y, int grid_z,
                           int block_x, int block_y, int block_z, void* stream);

/* The same with a status result, a thread-block-cluster width (0 = none) and dynamic shared memory. */
int cinn_b200_call_cuda_kernel_ex(void* kernel_fn, void* v_args, int num_args, int grid_x, int grid_y, int grid_z,
                                  int block_x, int block_y, int block_z, unsigned cluster_x, size_t dyn_smem,
                                  void* stream);

/*
 * Prebuilt-kernel table.  Replaces CUDAModule::GetFunction (cinn/runtime/cuda/cuda_module.cc:73-101) and
 * the JIT symbol registration of cinn/runtime/cuda/cuda_intrinsics.cc:404-418: kernels are compiled
 * offline for sm_100a and found by name.
 */
void* cinn_b200_get_kernel(const char* kernel_name);
int cinn_b200_num_kernels(void);
const char* cinn_b200_kernel_name(int index);
int cinn_b200_kernel_num_params(const char* kernel_name);

/* Number of kernel launches issued by this library in the calling process so far. */
long long cinn_b200_launch_count(void);

/* ---- fused groups ------------------------------------------------------------------------------- */

/*
 * Compile one fused group to a launch plan over the prebuilt kernels and bind it to an entry point of the
 * reference's type.  The group is given as text, one item per line:
 *     group <function name>
 *     input <id> <dtype> <d0,d1,...>                       (one per input, in argument order)
 *     op <HLIR op name> <out id> = <in id> ... ; key=value ...   (topological order, the reference's attributes)
 *     output <id> <dtype> <d0,d1,...>
 * The result is bound to an entry point of the reference's
 * type lower_func_ptr_g (cinn/runtime/cinn_runtime.h:497-499).  Replaces, for the groups it covers,
 * ParallelCompiler::Task::Lowering + CodegenAndJit (cinn/hlir/framework/parallel_compiler.cc:123-199).
 * The entry point takes cinn_pod_value_t[num_args] = the group's inputs then outputs, each a
 * cinn_buffer_t* holding device memory (cinn/hlir/framework/instruction.cc:81-105), and a CUstream.
 * Compiling the same name again replaces the earlier plan.  Needs no GPU.
 */
int cinn_b200_compile_group(const char* group_desc, lower_func_ptr_g* fn_out);

/* By-name lookup, as backends::ExecutionEngine::Lookup (cinn/backends/llvm/execution_engine.cc:221-230)
 * does for Instruction construction (cinn/hlir/framework/parallel_compiler.cc:201-217). NULL if unknown. */
lower_func_ptr_g cinn_b200_lookup(const char* fn_name);

/* Forget a compiled group and free its device scratch. */
int cinn_b200_release_group(const char* fn_name);

/* What lower_func_ptr_g does, with a status result instead of the last-error side channel. */
int cinn_b200_group_run(const char* fn_name, void* pod_args, int num_args, void* stream);

/* Facts about a compiled group: matched kernel family, bytes of inputs+outputs, elements, launches per run,
 * device scratch bytes.  Any out pointer may be NULL. */
int cinn_b200_group_info(const char* fn_name, char* pattern, size_t pattern_len, long long* algorithmic_bytes,
                         long long* elements, int* launches, long long* scratch_bytes);

/* Name of the kernel of launch step `step` of a compiled group (for tests and profiles). */
int cinn_b200_group_kernel(const char* fn_name, int step, char* name, size_t name_len);

/* The launch plan of a compiled group as text, for tests, profiles and the generator of the build-time chain
 * kernels: one "launch <i> <kernel> grid=x,y,z block=x,y,z cluster=c smem=bytes" line per launch, each followed by
 * one "arg <k> input|output <index>" / "arg <k> int <value>" / "arg <k> float <value>" / "arg <k> scratch <offset>" /
 * "arg <k> aligned <0|1>" line per kernel parameter.  Written to `out` (truncated to out_len); returns the size
 * needed including the terminator, negative on error.  The reference's counterpart is the generated host stub
 * itself (cinn/backends/codegen_cuda_host.cc:35-170), which can only be read as LLVM IR. */
long long cinn_b200_group_launch_text(const char* fn_name, char* out, size_t out_len);

/* How many chain programs have a kernel specialised at build time in this library. */
int cinn_b200_num_static_chains(void);

/* The matcher's canonical expression of a group description, e.g. "relu(elementwise_add(%0,%1))". */
int cinn_b200_canonical_expr(const char* group_desc, char* out, size_t out_len);

/*
 * Run a compiled group on HOST buffers: every cinn_buffer_t in pod_args holds host memory (pinned for full
 * copy speed); inputs are copied to `device`, the group runs, outputs are copied back, and the call returns
 * after the outputs are complete.  This is the path Tensor::from_numpy -> Program::Execute -> Tensor::numpy
 * takes in the reference (cinn/frontend/computation.cc:186-240, cinn/pybind/framework.cc:116-172).
 * Device staging memory is kept per group and device and reused by later calls.  Groups that are independent
 * along their outer axis are pipelined over chunks of it (see cinn_b200_group_host_chunks).
 */
int cinn_b200_group_run_host(const char* fn_name, void* pod_args, int num_args, int device);

/* In how many chunks of the outer axis cinn_b200_group_run_host pipelines this group (host->device copy of one
 * chunk, kernel of another, device->host copy of a third overlap on three streams); 1 when the group's outer
 * axis cannot be sliced (a reduction over it, an operand aligned to it, scratch memory) or it is too small. */
int cinn_b200_group_host_chunks(const char* fn_name);

/* ---- NetBuilder / Computation --------------------------------------------------------------------- */

/*
 * Program construction, the C form of frontend::NetBuilder (cinn/frontend/net_builder.h:125-1146).  A variable
 * is named by its id string.  cinn_b200_builder_add_op is the generic form of every op method: `op_type` is the
 * HLIR op name (elementwise_add, relu, scale, cast, reduce_sum, softmax, batch_norm, ... as registered in
 * cinn/hlir/op/elementwise.cc:860-1066, broadcast.cc:361-441, reduction.cc:477-505, nn.cc:2262-2433), `attrs`
 * a blank-separated "key=value" list with the reference's attribute names (axis, scale, bias,
 * bias_after_scale, dtype, dim, keep_dim, epsilon, data_layout, out_shape, broadcast_axes, shape, value).
 * Output shape and dtype are inferred; the new variable's id is written to id_out.
 */
typedef struct cinn_b200_builder cinn_b200_builder;
cinn_b200_builder* cinn_b200_builder_create(const char* name);
void cinn_b200_builder_destroy(cinn_b200_builder* builder);
int cinn_b200_builder_create_input(cinn_b200_builder* builder, const char* dtype, const long long* shape, int ndim,
                                   const char* id_hint, char* id_out, size_t id_len);
int cinn_b200_builder_add_op(cinn_b200_builder* builder, const char* op_type, const char* const* input_ids,
                             int num_inputs, const char* attrs, char* id_out, size_t id_len);
int cinn_b200_builder_var_info(cinn_b200_builder* builder, const char* id, char* dtype, size_t dtype_len,
                               long long* shape /* [8] */, int* ndim);

/*
 * Program passes: replaces ProgramPass::Apply as reached from Program.apply_pass and Program.build_and_get_output
 * (cinn/frontend/program_pass.h:36-105, cinn/pybind/frontend.cc:157-242).  Rewrites the builder's instruction list in
 * place by the named passes, in order; num_passes == 0 applies the reference's default list
 * (cinn/frontend/optimize.cc:44-82).  Built: "AutoCast" (auto_cast.cc), "AutoBroadcast" (auto_broadcast.cc),
 * "CastCollapsing" (cast_collapsing.cc), "TransposeCollapsing" (transpose_collapsing.cc), "FillConstantRewriter",
 * "FillConstantFolding", "Decomposer" (gelu, softmax modes, inference batch_norm), "RemoveIdentity"
 * (remove_identity.cc), "DeadCodeEliminate"; the other names of
 * the default list are accepted and change nothing; any other name fails with CINN_B200_EINVAL.  `fetch_ids` are the
 * variables that must survive.  Variable ids handed out earlier stay valid.  program_text writes one line per
 * instruction ("op out = in, in ; attr=value ...") into `out` (truncated to out_len) and returns the size needed
 * including the terminator.
 */
int cinn_b200_builder_apply_passes(cinn_b200_builder* builder, const char* const* passes, int num_passes,
                                   const char* const* fetch_ids, int num_fetch);
long long cinn_b200_builder_program_text(cinn_b200_builder* builder, char* out, size_t out_len);

/*
 * CinnComputation (cinn/frontend/computation.h:26-158): BuildAndCompile runs the fusion pass (the counterpart of
 * OpFusionPass + FusionMergePass, cinn/hlir/pass/op_fusion_pass.cc:123-331), compiles every group to prebuilt
 * kernels and allocates the scope's tensors on `device` with cudaMalloc (device < 0: plan only, no GPU touched).
 * fetch_ids name the variables to materialise (none: every variable that nothing consumes).  NULL on failure.
 * Execute runs the groups in order on `stream` and, like Program::Execute (cinn/hlir/framework/
 * graph_compiler.cc:212-222), synchronises the device only when stream is NULL.  set/get_tensor_data copy
 * between host memory and a scope tensor (computation.cc:186-240); bind_tensor substitutes caller-owned device
 * memory for a scope tensor (the reference's external-buffer mode, graph_compiler.cc:1305-1398).
 */
typedef struct cinn_b200_computation cinn_b200_computation;
cinn_b200_computation* cinn_b200_computation_build_and_compile(cinn_b200_builder* builder, int device,
                                                               const char* const* fetch_ids, int num_fetch);
void cinn_b200_computation_destroy(cinn_b200_computation* computation);
/*
 * Ahead-of-time program: replaces Program::Export and the tiny runtime's loader
 * (cinn/hlir/framework/graph_compiler.cc:89-210, cinn/runtime/tiny_runtime.cc:40-136).  export writes the compiled
 * program as text (tensors, group descriptions in execution order, aliases) into `out` (truncated to out_len) and
 * returns the size needed including the terminator; program_load rebuilds a computation from that text with no
 * builder and no fusion pass (device < 0: plan only), NULL + last_error on failure.
 */
long long cinn_b200_computation_export(cinn_b200_computation* computation, char* out, size_t out_len);
cinn_b200_computation* cinn_b200_program_load(const char* text, int device);
int cinn_b200_computation_execute(cinn_b200_computation* computation, void* stream);
/* The whole program as one CUDA graph: captured at the first call (which also runs the program once the ordinary
 * way), replayed by later calls, re-captured after bind_tensor.  `stream` must not be NULL.  The reference has no
 * counterpart: its host loop issues one launch per instruction at every Execute. */
int cinn_b200_computation_execute_graph(cinn_b200_computation* computation, void* stream);
/* Program::ExecuteTest (cinn/hlir/framework/graph_compiler.cc:224-244): 100 untimed runs, then `repeat` runs timed on
 * the host clock up to a device synchronisation; writes the average milliseconds per run.  repeat < 0 measures
 * |repeat| replays of the program's CUDA graph instead. */
int cinn_b200_computation_execute_test(cinn_b200_computation* computation, int repeat, double* avg_ms);
int cinn_b200_computation_set_tensor_data(cinn_b200_computation* computation, const char* id, const void* host,
                                          size_t bytes);
int cinn_b200_computation_get_tensor_data(cinn_b200_computation* computation, const char* id, void* host,
                                          size_t bytes);
int cinn_b200_computation_bind_tensor(cinn_b200_computation* computation, const char* id, void* device_ptr);
int cinn_b200_computation_num_tensors(cinn_b200_computation* computation);
const char* cinn_b200_computation_tensor_name(cinn_b200_computation* computation, int index);
int cinn_b200_computation_tensor_info(cinn_b200_computation* computation, const char* id, char* dtype,
                                      size_t dtype_len, long long* shape /* [8] */, int* ndim, void** device_ptr);
/* 0: an input of the program (nothing in it writes the tensor), 2: an output (written, read by nothing in it),
 * 1: in between; negative on error.  What GetInputTensors / GetOutputTensors of frontend::CinnComputation
 * (cinn/frontend/computation.h:120-140) enumerate. */
int cinn_b200_computation_tensor_role(cinn_b200_computation* computation, const char* id);
/* The groups the fusion pass produced: description text, and "pattern kernel kernel ..." of the match. */
int cinn_b200_computation_num_groups(cinn_b200_computation* computation);
int cinn_b200_computation_group_desc(cinn_b200_computation* computation, int index, char* out, size_t out_len);
int cinn_b200_computation_group_pattern(cinn_b200_computation* computation, int index, char* out, size_t out_len);

/*
 * Column reduction without any allocation.  No counterpart in the reference (its kernels never need scratch
 * memory: it reduces such shapes with one serial loop per output element).
 *
 * y[o, i] = reduce over k of x[o, k, i], x viewed as [outer, r, inner] fp32, kind 0 sum / 1 prod / 2 max / 3 min:
 * the same kernels and the same two-step split over r as a compiled reduce group uses, but the partials go to a
 * fixed 4 MiB array inside the library instead of scratch obtained with cudaMalloc.  It exists for callers that
 * must not have this library allocate device memory: a host framework that owns the whole device pool and passes
 * in only buffers of its choosing, or a serving loop where the device-wide synchronisation of a cudaMalloc is
 * not acceptable.  x and y are device pointers supplied by the caller; the call issues one or two launches on
 * `stream` and returns without synchronising.
 *
 * Limits and rules: two partials of the output must fit the static array: 2 * outer * inner <= 1,048,576 floats.
 * Any larger output is refused with CINN_B200_ENOSPACE and a message, whether or not this device would split the
 * reduced axis for it (so the limit does not depend on the SM count); such reductions run through a compiled
 * group, which needs no scratch when it does not split.  The first call
 * on each device looks up the array's device address (cudaGetSymbolAddress); make that first call outside any
 * stream capture.  All calls share the array, so calls that can overlap on the GPU (different streams or threads)
 * must be serialised by the caller.  Nothing needs to be cleared between calls.
 */
int cinn_b200_col_reduce_f32_static_scratch(int kind, const float* x, float* y, long long outer, long long r,
                                            long long inner, void* stream);

/* ---- reductions over an axis sharded across GPUs --------------------------------------------------- */

/*
 * No counterpart in the reference (it has no multi-GPU execution).  x is [R, inner] fp32 with the R axis split over
 * `world` ranks, one process per GPU of one node; every rank holds rows_local rows.  One kernel per rank reduces the
 * local rows and exchanges the partials over NVLink peer memory (plain peer stores, mapped with CUDA IPC; no
 * multicast): each rank ends up with the final result of the band of columns it owns (all_gather == 0: `out` holds
 * inner / world elements, band `rank`) or with the full result (all_gather != 0: `out` holds inner elements).
 * Requirements: inner % (4 * world) == 0, 16-byte aligned x_local / out, every rank calls with the same kind /
 * inner / all_gather, in the same order, and a context serves ONE inner size and ONE result mode (fixed by its first
 * call).  A result whose bits are 0xFFFFFFFF (a NaN pattern used inside as "not arrived") is delivered as the default
 * NaN 0x7FFFFFFF.  Waits on peers are bounded (about a quarter of a second); a wait that runs out is reported by
 * cinn_b200_device_status and cinn_b200_peer_status, leaves `out` undefined and the context unusable (destroy it).
 *
 * peer_create allocates this rank's exchange buffer for results of up to max_inner elements and writes its 64-byte
 * IPC handle; the caller gathers the handles of all ranks (rank order) and passes them to peer_connect.
 *
 * Teardown has two steps with a barrier between them, because CUDA leaves freeing an exported allocation while
 * another process still has it open undefined: every rank calls peer_close_imports (which first waits for this
 * rank's device to go idle), the caller runs a barrier over all ranks, then every rank calls peer_destroy.
 * peer_destroy alone closes the imports too, for a world of one or when the caller has synchronised the ranks itself.
 *
 * The ranks' launches of one call must start within the wait budget of each other (about a quarter of a second);
 * a first call delayed by a module load or a stalled host on one rank can exhaust it on all.  After a wait has run
 * out the context stays failed: later launches on it return at once without touching `out`, peer_status writes 1.
 */
typedef struct cinn_b200_peer_ctx cinn_b200_peer_ctx;
int cinn_b200_peer_create(int rank, int world, long long max_inner, unsigned char* handle_out /* 64 bytes */,
                          cinn_b200_peer_ctx** ctx_out);
int cinn_b200_peer_connect(cinn_b200_peer_ctx* ctx, const unsigned char* all_handles /* world * 64 bytes */);
int cinn_b200_peer_close_imports(cinn_b200_peer_ctx* ctx);
int cinn_b200_peer_destroy(cinn_b200_peer_ctx* ctx);
/* 1 in *failed_out when a bounded wait of an earlier call on this context gave up (synchronises with the device). */
int cinn_b200_peer_status(cinn_b200_peer_ctx* ctx, int* failed_out);
int cinn_b200_col_reduce_sharded_f32(cinn_b200_peer_ctx* ctx, int kind /* 0 sum, 1 prod, 2 max, 3 min */,
                                     const float* x_local, long long rows_local, long long inner, float* out,
                                     int all_gather, void* stream);

/*
 * The same kernel with every rank of the world on ONE GPU: peer_create_emulated allocates `world` exchange buffers
 * on the current device, and one launch (gridDim.y = world) runs all ranks at once, rank r reading x_per_rank[r]
 * ([rows_local, inner]) and writing out_per_rank[r].  It exists so that the exchange protocol -- arrival by
 * sentinel, rank-order combination, the three rotating areas -- can be verified on a machine with a single GPU; the
 * stores that cross NVLink in the real form are local stores here.  Destroy with peer_destroy.  No counterpart in
 * the reference.
 */
int cinn_b200_peer_create_emulated(int world, long long max_inner, cinn_b200_peer_ctx** ctx_out);
int cinn_b200_col_reduce_sharded_f32_emulated(cinn_b200_peer_ctx* ctx, int kind, const float* const* x_per_rank,
                                              long long rows_local, long long inner, float* const* out_per_rank,
                                              int all_gather, void* stream);
/*
 * The emulated launch restricted to ranks rank0 .. rank0 + nranks - 1 (the arrays are still indexed by rank; only
 * those entries are read).  With fewer ranks than the world, the launched ranks wait for partials that never come:
 * their bounded waits run out after about a quarter of a second, the call counts as failed
 * (cinn_b200_device_status, cinn_b200_peer_status) and later calls on the context return without touching `out`.
 * This is how the give-up path is exercised without a second GPU or a process that dies.
 */
int cinn_b200_col_reduce_sharded_f32_emulated_ranks(cinn_b200_peer_ctx* ctx, int kind, const float* const* x_per_rank,
                                                    long long rows_local, long long inner, float* const* out_per_rank,
                                                    int all_gather, int rank0, int nranks, void* stream);

/*
 * Device-side status of the current device: the number of bounded waits on asynchronous copies that gave up
 * since the last call (0 in a healthy run); reading clears it.  Synchronises with the device.  The reference
 * has no counterpart (its generated kernels never wait on asynchronous copies).
 */
int cinn_b200_device_status(unsigned int* async_wait_timeouts);

/* Tuning knobs (integers) read by the matcher when a group is compiled; unknown keys give CINN_B200_ENOTFOUND.
 * "sm_count": SM count assumed when no GPU is visible (default 148); "enable_pdl" (default 1; read at every launch):
 * kernels that wait for their predecessor on the device are launched with programmatic stream serialisation, which
 * hides the launch latency between consecutive kernels of a stream; "enable_static_chains" (default 1): elementwise
 * chains whose program has a kernel specialised at build time use it instead of the interpreting kernel;
 * "fuse_interpreted_programs" (default 0): the fusion pass also forms groups that only the interpreting register-program
 * or row-program kernel takes (one launch, but several times slower per byte than the specialised kernels; off, such
 * regions are split into groups the chain and reduction kernels take; a group handed to cinn_b200_compile_group
 * directly is always accepted);
 * "peer_reducers_per_sm" (default 0 = as many as fit): the most reducer CTAs per SM of the fused reduce + exchange
 * kernel (fewer reducers take their items in more rounds; measured on 4 GPUs: two to four per SM change nothing, one
 * per SM is too few to stream the local rows at full bandwidth);
 * "host_chunks" (default 0 = up to 16): the most chunks cinn_b200_group_run_host pipelines a group over (read at the
 * group's first host run);
 * "rowp_form" (default 0 = automatic): the form of a row program -- 32 a warp per row, 128 half a CTA per row
 * (specialised kernels only), 256 a CTA per row;
 * "ew_reg_ctas_per_sm" (default 0 = by size): grid of the register form of the bias / scale / tanh / cast kernel in
 * CTAs per SM (measured on an 8.4 M-element shard: 4 to 16 per SM all within 10.7-11.2 us);
 * "enable_ew_stream" (default 1),
 * "ew_stream_stages", "ew_stream_ctas_per_sm": whether large elementwise groups with 16-bit outputs stream their
 * input through shared-memory rings filled by bulk copies, the ring depth and the resident CTAs per SM; "rownorm_rows_per_iter": rows per CTA
 * iteration of the register-resident softmax / layer_norm kernels (0 = automatic, else 1, 2 or 4); "rownorm_stages", "rownorm_ctas_per_sm":
 * ring depth and resident CTAs per SM of the streamed softmax / layer_norm kernels (0 = automatic);
 * "enable_tma_rownorm": 1 selects the kernels that stream rows through a shared-memory ring with bulk
 * asynchronous copies, 0 the register-resident ones, -1 (default) chooses per group; "rownorm_simple": 1 runs the
 * plain softmax through the one-CTA-per-row kernel written for the max-subtracted form (measured equal; default off). */
int cinn_b200_set_option(const char* key, long long value);

#ifdef __cplusplus
}
#endif

#endif /* CINN_B200_H_ */
