/* C-ABI of libhc-b200-kernels.so: the precompiled sm_100a kernel images and
 * one launch entry point per workload.
 *
 * In the reference a kernel reaches the GPU as a binary blob that JIT-compiled
 * host code hands to hcgpuGetKernel / hcgpuLaunchKernel
 * (python/cpp/py-runtime/src/GpuRuntime.cpp:26-69) and from there to the ol*
 * ABI (gpu-runtime/common/include/offload_api.h:29-63).  This library takes
 * the place of that JIT-compiled host code: it owns the blobs (now cubins
 * built ahead of time), picks the kernel variant for the argument shapes,
 * packs the kernel parameters and launches through the same ol* ABI of the
 * loader (olCreateModule / olGetKernel / olLaunchKernel).  It never computes
 * on the host and has no fallback when no GPU is present.
 *
 * All pointers are device pointers unless stated otherwise; pitches are in
 * elements; every launch is asynchronous on the context's queue.  Functions
 * returning int return 0 on success; on failure they return nonzero, call the
 * context's OlErrorCallback and keep the text for hcLastError.
 */
#pragma once

#include "offload_api.h"

#ifdef __cplusplus
extern "C" {
#endif

#define HC_B200_API __attribute__((visibility("default")))

typedef struct HcContextImpl *HcContext;

/* Element types of the workload entry points. */
enum HcDType {
  HC_F32 = 0,
  HC_F64 = 1,
  HC_BF16 = 2,
  HC_I8 = 3,
  HC_I32 = 4,
  HC_I64 = 5
};

/* ---- kernel images -------------------------------------------------------
 * The blobs a caller would pass to olCreateModule / hcgpuGetKernel, replacing
 * the output of the reference's gpu-module-to-binary step
 * (mlir/lib/Pipelines/BackendPipeline.cpp:55-61). */
HC_B200_API int hcImageCount(void);
HC_B200_API const char *hcImageName(int index);
HC_B200_API const void *hcImageData(int index, size_t *lenRet);
/* Image that defines `kernelName`, or -1. */
HC_B200_API int hcImageOfKernel(const char *kernelName);

/* ---- context: device + queue + loaded images ------------------------------
 * Plays the role of the process-global device/queue pair of the reference's
 * py-runtime (GpuRuntime.cpp:23-39), but one per device description so that
 * several GPUs can be driven from one process.  Like the reference's runtime
 * (no locks anywhere, gpu-runtime/cuda-runtime/src/Runtime.cpp), a context is
 * not thread-safe: use it from one thread at a time.  Different contexts may
 * be used from different threads. */
HC_B200_API HcContext hcCreateContext(const char *deviceDesc,
                                      OlErrorCallback errCallback, void *ctx);
HC_B200_API void hcReleaseContext(HcContext c);
HC_B200_API OlDevice hcContextDevice(HcContext c);
HC_B200_API OlQueue hcContextQueue(HcContext c);
/* The CUstream behind the context's queue. */
HC_B200_API void *hcContextStream(HcContext c);
HC_B200_API int hcSynchronize(HcContext c);
HC_B200_API const char *hcLastError(HcContext c);
/* Kernel launches issued through this context so far. */
HC_B200_API long long hcLaunchCount(HcContext c);
/* Synchronizes, then returns in *statusRet the status word the tensor-core
 * kernels write when one of their bounded waits gives up (0 = none did) and
 * clears it. */
HC_B200_API int hcKernelStatus(HcContext c, int *statusRet);
/* Runs a one-CTA kernel whose barrier wait can never be satisfied, with the
 * given time limit, waits for it and returns what happened: the status word
 * it published (expected 1, "producer wait"), how long the kernel was inside
 * (nanoseconds), and whether its two waiting threads saw their waits succeed
 * (expected 0 and 0: one ran out of time, the other left on the abort flag).
 * Exercises, without any fault, the mechanism that keeps a protocol bug in the
 * TMA/tcgen05 kernels from hanging the GPU.  No counterpart in the reference. */
HC_B200_API int hcSelfTestWaitTimeout(HcContext c, unsigned long long limitNs,
                                      int *statusRet,
                                      unsigned long long *elapsedNsRet,
                                      int observedRet[2]);

/* Tuning and test switches.  "gemm_variant": 0 = automatic, 1 = one CTA per
 * tile, 2 = CTA pair per tile, 3 = CUDA-core tiled kernel.  "tiled_variant"
 * (fp32 hcGemmTiled): 0 = automatic, 1 = no cp.async pipeline, 2 = pipeline
 * but no split of K over a cluster.  "mapped_stack":
 * 0 = hcMappedGemm stacks work-groups that share their f tile (up to 128 rows
 * of float tiles wider than 16 columns, else 64), 1 = one work-group per CTA,
 * 2 = stacks of at most 64 rows.  "row_variant" (hcRowProgram): 0 = float rows of 257..1024
 * 16-byte packets that fill at least 90 % of a CTA of 64 or 128 threads are held in the
 * registers of one CTA per row (eight packets per thread on 64, 96 or 128
 * threads), 1 = always one warp per row that walks the row once per pass,
 * 2 = as 3, with 256 threads and four packets each beyond 512 packets,
 * 3 = hold such rows whatever the fill.  "fused": 0 = programs that match a body
 * compiled ahead of time run as straight-line kernels, 1 = every program is
 * interpreted.  "specialise": what happens to a program of hcMapElements /
 * hcRowProgram that has no such body, and to every program of hcWorkItems - 1 (default) = it is compiled at its first
 * launch (see hcSpecialisedPrograms) and interpreted where that is not possible,
 * 0 = it is interpreted, 2 = as 1, but the launch fails where compiling is not
 * possible.  "conv_variant" (hcConvF32Tensor): 0 = the library's choice - with
 * stride 1 both operands come by TMA (4 where two of its stages fit in shared
 * memory, else 3), otherwise threads gather the image operand (2 where at most
 * 128 filters leave room in tensor memory, else 1); 1 = gathered into shared
 * memory, 2 = gathered into tensor memory (more filters are refused), 3 = by
 * TMA, a rectangle of 128 pixels per filter tap, 4 = by TMA, runs of 128
 * positions of the flattened image, the patch of a filter row shared by its
 * taps; 3 and 4 take stride 1 and fail on images too small for their boxes.
 * "conv_stages": 0 or 2..6 pipeline stages; "conv_stacked": 0 = with at
 * most 128 filters the two products that share a_hi run as one MMA of double
 * width, 1 = three MMAs per K step throughout.  "gemm_band": row tiles per
 * band in the tile order of the tcgen05 GEMMs (0 = 16).  "w8a16_variant"
 * (hcGemmW8A16): 0 and 1 = the weights are converted by a pass of their own into
 * the workspace, 2 = inside the GEMM's pipeline (no workspace), 3 = inside the
 * GEMM kernel band by band into a ring of three bands (hcGemmW8A16BandedBytes of
 * workspace); 2 and 3 fail where the layout does not allow them, and all give
 * the same result bit for bit. */
HC_B200_API int hcSetOption(HcContext c, const char *name, long long value);

/* Run-time specialisation.  The reference compiles every kernel body at its
 * first call and keeps the result per argument signature
 * (python/cpp/native/DispatcherBase.cpp:250-256,542-585).  Here a program of
 * hcMapElements (any operation; float32, float64, int32, int64) or hcRowProgram
 * (float32, float64) that has no body compiled ahead of time is compiled the
 * first time a context launches it: NVRTC (looked up with dlopen; libnvrtc.so.12, or the
 * path in HC_B200_NVRTC) turns the kernel templates, embedded in this library as
 * text, into straight-line code for the program's instruction words; the image
 * is loaded and kept until the context is released.  Constants stay launch
 * parameters, so bodies that differ in constants alone share one image.  Results
 * equal the interpreter's bit for bit.  The first launch takes the time of the
 * compilation (about half a second); with HC_B200_KERNEL_CACHE naming a
 * directory, images are also kept there and later processes load them instead.
 * hcSpecialisedPrograms: how many programs this context compiled (fromDisk = 0)
 * or loaded from the directory (1).  hcSpecialiseNote: why the latest attempt
 * failed ("" if none did; the string lives until the next attempt). */
HC_B200_API long long hcSpecialisedPrograms(HcContext c, int fromDisk);
HC_B200_API const char *hcSpecialiseNote(HcContext c);

/* ---- workloads -------------------------------------------------------------
 * 2-D copy; the reference's compiled copy kernels
 * (python/hckernel/tests/test_e2e.py:57-136). */
HC_B200_API int hcCopy2D(HcContext c, const void *src, void *dst,
                         long long rows, long long cols, long long srcPitch,
                         long long dstPitch, int elemBytes);

/* Element-wise expression: out[r,c] = f(in0[r,c], ..., in3[r,c]) over
 * rows x cols matrices, HC_F32, HC_F64, HC_I32 or HC_I64 (all arrays one type).  What
 * work-groups compute that load tiles at one origin, combine them element by
 * element and store the result there - the reference's copy kernels
 * (python/hckernel/tests/test_e2e.py:57-136) with tile arithmetic
 * (python/hckernel/kernel_api.py:136-211) in between.  The reference compiles
 * such a body; here f is data: a program for a machine with one accumulator and
 * three temporaries.  An instruction is `op | (src << 8)`:
 *   op   0 load  1 add  2 sub  3 rsub (v - acc)  4 mul  5 div  6 rdiv (v / acc)
 *        7 max  8 min  9 neg  10 abs  11 exp  12 sqrt  13..15 save to t0..t2
 *        16 log
 *        the rest of the reference's tile operator table
 *        (python/hckernel/kernel_api.py:157-176), hcMapElements only:
 *        20 floordiv  21 rfloordiv (v // acc)  22 mod  23 rmod  24 pow  25 rpow
 *        26 lt  27 le  28 eq  29 ne  30 ge  31 gt   (acc = acc OP v ? 1 : 0)
 *        32 and  33 or  34 xor   (integers: bitwise; floats: logical on zero / nonzero)
 *        35 shl  36 shr  37 rshl (v << acc)  38 rshr   (integers only)
 *        39 inv   (integers: ~acc; floats: acc == 0 ? 1 : 0)
 *   src  0..3 input arrays, 4..6 temporaries t0..t2, 8..15 consts[0..7],
 *        16 / 17 the row / column index of the element, as a value (what a body
 *        written at work-item level gets from global_id(),
 *        python/hckernel/kernel_api.py:243-252, 395-414)
 * max and min give NaN when either operand is NaN (NumPy's maximum/minimum);
 * operations are never contracted into FMAs; integer arithmetic wraps; floor
 * division and remainder follow NumPy's (Python's sign conventions).  Integer
 * arrays take no division, exp, sqrt or log, integral constants only, and
 * constant non-negative exponents.  The value of the accumulator after the last
 * instruction is stored - except where the arithmetic made it invalid the way
 * NumPy's masked arrays mask an element (the reference's tiles are numpy.ma
 * arrays): a zero divisor of / // %, a power that is not finite.  Such elements
 * of `out` are left as they were, like the reference's masked store
 * (python/hckernel/kernel_api.py:338-340).  A program that matches one of the
 * bodies compiled ahead of time (hc_b200/csrc/kernels/fused_programs.h) runs as
 * a straight-line kernel, any other is interpreted; the results are the same
 * bit for bit.  Pitches are in elements. */
typedef struct HcMapProgram {
  const void *in[4];      /* device */
  long long inPitch[4];
  void *out;              /* device */
  long long outPitch;
  long long rows, cols;
  int nInputs;            /* 0..4 */
  int nInstr;             /* 1..32 */
  unsigned code[32];
  double consts[8];
} HcMapProgram;
HC_B200_API int hcMapElements(HcContext c, const HcMapProgram *program, int dtype);

/* Row program: out[r,:] = f(in0[r,:], in1[r,:]) where f may reduce along the
 * row and use the reduced values again - the reference's row softmax
 * (python/hckernel/tests/test_examples.py:312-321) generalised to any such
 * expression (centring, normalising, scaling rows by their own statistics).
 * Same program structure as hcMapElements (1 or 2 inputs, op 16 = log), with
 *   op   17 rsum / 18 rmax: end a pass over the row, reduce the accumulator
 *        along it into row scalar s[src], src 0..3 (max gives NaN if the row
 *        holds one); the next instruction must be a load
 *   src  20..23 the row scalars s0..s3, once reduced or set
 * A pass may open with uniform instructions - operation byte | 0x80 - that work
 * on one value per row (operands: constants and row scalars) and run once per
 * row instead of once per element; such a sequence starts with a load and ends
 * with op 19 set: s[src] = that value (the log of a sum, a mean from a sum).
 * The program must end with a pass that is not a reduction: its accumulator is
 * stored.  Temporaries do not carry over from one pass to the next; element
 * indices (src 16/17) are not available. */
HC_B200_API int hcRowProgram(HcContext c, const HcMapProgram *program, int dtype);

/* The compilation alone, without a context or a GPU (to fill the directory of
 * HC_B200_KERNEL_CACHE ahead of time, or to check that NVRTC is usable): the
 * device image of `program` (rowProgram: 0 = for hcMapElements, 1 = for
 * hcRowProgram; dtype as the entry point takes it) for compute capability
 * ccMajor.ccMinor.
 * Returns the size of the image and copies up to `capacity` bytes of it to `image`
 * (which may be null); `message` receives the tag that stands for the program in
 * the kernel names (hc_map_fused_<tag>_f32_v4 ...).  On failure returns -1 and
 * `message` says why.  No counterpart in the reference, whose compiler is not
 * reachable without its Python front end. */
HC_B200_API long long hcSpecialiseCompile(const HcMapProgram *program, int rowProgram,
                                          int dtype, int ccMajor, int ccMinor, void *image,
                                          size_t capacity, char *message,
                                          size_t messageCapacity);

/* Work-item program: a body written at work-item level
 * (CurrentGroup.workitems, python/hckernel/kernel_api.py:395-414) that an
 * element-wise pass cannot express - it uses the work-item's local id, reads a
 * neighbour's element, or has two phases separated by group.barrier()
 * (kernel_api.py:416-431) that exchange values through a tile of the work-group.
 * One thread per work-item, one CTA per work-group of groupRows x groupCols
 * (at most 1024 work-items), the tile in shared memory.  The program uses the
 * operations of hcMapElements on single values (no validity tracking: a zero
 * divisor gives the IEEE result), with an instruction `op | (src << 8)` and
 *   op   64 store to the group's tile at the work-item's local id
 *        65 barrier   66 store to out at the work-item's global id
 *   src  0..3 input k at (row + inRow[k], col + inCol[k]), 4..6 temporaries,
 *        8..15 constants, 16 / 17 global row / column, 18 / 19 local row / column,
 *        24..27 the tile at local index (tileScale * local id + tileOffset) mod
 *        tileMod per axis (tileMod 0: no wrap), table entry src - 24
 * A work-item takes part in phase p (0 before the barrier, 1 after it) only if
 * guardLo[p] <= global id < guardHi[p] on both axes - the `if gid < n` of the
 * body; all arrays are rows x cols (rows = 1 for one-dimensional work) and the
 * guards are cut to that.  HC_F32 or HC_F64. */
typedef struct HcItemProgram {
  const void *in[4];      /* device */
  long long inPitch[4];
  int inRow[4], inCol[4];
  void *out;              /* device */
  long long outPitch;
  long long rows, cols;
  int groupRows, groupCols;
  int nInputs;            /* 0..4 */
  int nInstr;             /* 1..48 */
  unsigned code[48];
  double consts[8];
  long long guardLo[2][2], guardHi[2][2]; /* [phase][0 rows, 1 columns] */
  int tileScale[4][2], tileOffset[4][2], tileMod[4][2];
  double tileFill;        /* the tile's content before the first store */
} HcItemProgram;
HC_B200_API int hcWorkItems(HcContext c, const HcItemProgram *program, int dtype);

/* hcSpecialiseCompile for a work-item program: `code` holds the nInstr
 * instruction words of an HcItemProgram, dtype HC_F32 or HC_F64, groupThreads the
 * work-group size (groupRows * groupCols) the kernel is to serve: work-groups of
 * up to 256 work-items get a kernel that keeps 32 bytes of loads in flight per
 * thread, larger ones a kernel within the register budget of 1024 threads.  The
 * kernel of the image is hc_work_items_fused_<tag>_f32 or _f64.  hcWorkItems
 * compiles its program the same way at the first launch, under the option
 * `specialise`. */
HC_B200_API long long hcSpecialiseCompileItems(const unsigned *code, int nInstr, int dtype,
                                               int groupThreads, int ccMajor, int ccMinor,
                                               void *image,
                                               size_t capacity, char *message,
                                               size_t messageCapacity);

/* Row softmax over the last axis, HC_F32 or HC_F64
 * (python/hckernel/tests/test_examples.py:304-321). */
HC_B200_API int hcSoftmaxRows(HcContext c, const void *x, void *y,
                              long long rows, long long cols, long long xPitch,
                              long long yPitch, int dtype);

/* Last-axis sum and/or max (either output may be NULL), HC_F32 or HC_F64
 * (python/hckernel/tests/test_examples.py:31-71 for the sum form). */
HC_B200_API int hcReduceRows(HcContext c, const void *x, void *sumOut,
                             void *maxOut, long long rows, long long cols,
                             long long pitch, int dtype);

/* ---- compute and all-gather in one kernel (multi-GPU) ---------------------------
 * In a job with one process per GPU every rank computes its rows of the result
 * and all ranks need the whole of it.  Instead of computing into local memory
 * and running an all-gather afterwards, these variants write every result row
 * straight into the full output buffer of EVERY rank: `dsts->base[d]` is where
 * this rank's row 0 goes in rank d's buffer (its own included) - device memory
 * of this GPU or peer memory of another GPU mapped into this process (CUDA IPC,
 * torch symmetric memory).  Plain stores over NVLink; no kernel waits for
 * another, so nothing can hang: the caller orders the ranks afterwards (any
 * cross-rank barrier on the stream) before anyone reads the buffers.  No
 * counterpart in the reference, which drives one device per process
 * (python/cpp/py-runtime/src/GpuRuntime.cpp:23-24).
 *
 * hcSoftmaxRowsPeers: float32 rows of at most 4096 columns, a multiple of 4,
 * 16-byte aligned bases and pitches (the register kernel of hcSoftmaxRows).
 * hcReduceRowsPeers: sums to base[d][r], maxima to base[d][maxOffset + r]. */
typedef struct HcPeerOutputs {
  void *base[8];
  int count; /* 1..8 */
} HcPeerOutputs;
HC_B200_API int hcSoftmaxRowsPeers(HcContext c, const void *x, const HcPeerOutputs *dsts,
                                   long long rows, long long cols, long long xPitch,
                                   long long yPitch, int dtype);
HC_B200_API int hcReduceRowsPeers(HcContext c, const void *x, const HcPeerOutputs *dsts,
                                  long long maxOffset, long long rows, long long cols,
                                  long long pitch, int dtype);

/* The tensor-core GEMMs with the same kind of output (hcGemmBf16 / hcGemmW8A16
 * otherwise): base[d] is where element [0, 0] of this call's output block goes
 * in rank d's copy of C, `ldc` the pitch of the full C - an M-shard passes its
 * row block's address, an N-shard its column block's.  Operands that the
 * tensor-core kernel cannot take are refused (there is no CUDA-core form). */
HC_B200_API int hcGemmBf16Peers(HcContext c, const void *a, const void *b,
                                const HcPeerOutputs *dsts, long long M, long long N,
                                long long K, long long lda, long long ldb, long long ldc);
HC_B200_API int hcGemmW8A16Peers(HcContext c, const void *a, const void *w,
                                 const float *scale, const HcPeerOutputs *dsts,
                                 void *workspace, size_t workspaceBytes, long long M,
                                 long long N, long long K, long long lda, long long ldw,
                                 long long ldc);

/* Whole-array sum added to one element: result[0] += sum(a[0:n]).  `a` is
 * HC_F32, HC_F64, HC_I32 or HC_I64; `result` is HC_F32 or HC_F64 and is not
 * cleared first (the reference's atomic_ref(result)[0] += tile.sum(),
 * python/hckernel/tests/test_examples.py:31-71). */
HC_B200_API int hcReduceAll(HcContext c, const void *a, long long n,
                            void *result, int inDtype, int resultDtype);

/* Pairwise Euclidean distance: out[i,j] = sqrt(sum_d (a[i,d] - b[j,d])^2) for
 * a [M,D], b [N,D], out [M,N]; HC_F32 or HC_F64
 * (python/hckernel/tests/test_examples.py:261-301). */
HC_B200_API int hcPairwiseDistance(HcContext c, const void *a, const void *b,
                                   void *out, long long M, long long N,
                                   long long D, long long lda, long long ldb,
                                   long long ldo, int dtype);

/* Gathered tile product: what work-groups compute that load their operand tiles
 * with group.load(view, shape, mapping=...), multiply them and write the result
 * with group.store(view, tile, mapping=...)
 * (python/hckernel/kernel_api.py:297-336; the implicit-GEMM convolution of
 * python/hckernel/tests/test_examples.py:203-252).  For every work-group g
 *   A[a,k] = x[xOrigin(g) + xMap(a,k)],  B[k,b] = f[fOrigin(g) + fMap(k,b)]
 *   out[oOrigin(g) + oMap(a,b)] = sum_k A[a,k] * B[k,b]
 * where an operand element whose mapped index falls outside its array reads as
 * zero and a result element whose mapped index falls outside `out` is dropped.
 * The mappings arrive as tables in device memory, evaluated by the caller:
 *   map      int32 [tile elements][4]  mapped index relative to the tile origin
 *   lin      int32 [tile elements]     sum_d map[d] * stride[d]
 *   origins  int32 [groups][4]         tile origin of every work-group (>= 0)
 * with tile elements in row-major order of the tile ([TM,K], [K,TN], [TM,TN])
 * or, for x and f, transposed ([K,TM], [TN,K]) when `transposed` is set: the
 * kernel hands consecutive table entries to consecutive threads, so the caller
 * picks the order in which neighbouring entries are neighbours in memory.
 * `map` and `origins` must be 16-byte aligned.  Arrays of rank below 4 are
 * padded with shape 1, stride 0 and zeros in the tables.  lo/hi are the
 * smallest/largest value of each column of `map`.  Distinct (group, element)
 * pairs must not map to the same element of `out`, and `out` must not overlap
 * x or f.  HC_F32 or HC_F64. */
typedef struct HcMappedOperand {
  void *base;           /* device: element [0,0,0,0] of the array */
  const int *map;       /* device */
  const int *lin;       /* device */
  const int *origins;   /* device */
  int shape[4];
  long long stride[4];  /* in elements */
  int lo[4];
  int hi[4];
  int transposed;       /* order of map/lin; must be 0 for out */
  int sharedRun;        /* n > 1: work-groups g with equal g / n have the same
                           origin in this array (read for f only: such groups
                           use one f tile, so one CTA computes several of them
                           against it); 0 or 1: nothing known */
} HcMappedOperand;
HC_B200_API int hcMappedGemm(HcContext c, const HcMappedOperand *x,
                             const HcMappedOperand *f, const HcMappedOperand *out,
                             long long groups, int TM, int TN, int K, int dtype);

/* C[M,N] = A[M,K] @ B[K,N] on the CUDA cores; HC_F32, HC_F64, or HC_BF16
 * (bf16 in and out, fp32 accumulation)
 * (python/hckernel/tests/test_examples.py:74-165). */
HC_B200_API int hcGemmTiled(HcContext c, const void *a, const void *b, void *cOut,
                            long long M, long long N, long long K,
                            long long lda, long long ldb, long long ldc,
                            int dtype);

/* float32 GEMM on the tensor cores: C[M,N] = A[M,K] @ B[K,N], float32 in and
 * out, for the same dot kernels as hcGemmTiled
 * (python/hckernel/tests/test_examples.py:74-165) at sizes where the CUDA cores
 * are the limit.  Every operand is split into two tf32 numbers and three tf32
 * products per product accumulate in fp32 (tcgen05.mma.kind::tf32), which keeps
 * the result within about 3e-7 * sum|a||b| of the exact one - float32 class,
 * where a single tf32 product would lose three digits.  `workspace` must hold
 * hcGemmF32TensorWorkspaceBytes(M, N, K) bytes of device memory, 1 KiB aligned
 * (the split operands); it is written by every call.  On a device without
 * tcgen05, or with "gemm_variant" 3, the call runs hcGemmTiled instead. */
HC_B200_API size_t hcGemmF32TensorWorkspaceBytes(long long M, long long N, long long K);
HC_B200_API int hcGemmF32Tensor(HcContext c, const void *a, const void *b, void *cOut,
                                void *workspace, size_t workspaceBytes, long long M,
                                long long N, long long K, long long lda, long long ldb,
                                long long ldc);

/* float32 convolution on the tensor cores, without padding:
 *   out[n, q, oh, ow] = sum over (c, kh, kw) of
 *       x[n, c, oh * stride + kh, ow * stride + kw] * f[q, c, kh, kw]
 * x [N, C, H, W], f [NF, C, HF, WF], out [N, NF, HO, WO] with
 * HO = (H - HF) / stride + 1 and WO = (W - WF) / stride + 1, all float32 and
 * contiguous.  The sums of the reference's implicit-GEMM convolution
 * (python/hckernel/tests/test_examples.py:203-252) for square outputs, tiled by
 * output pixels instead of by (images x filters) per position: an implicit GEMM
 * whose products run as three tf32 products each on tcgen05 (float32-class
 * results, as hcGemmF32Tensor).  With stride 1 the image is rewritten once with
 * the channels innermost and both operands reach the MMA by TMA; with other
 * strides the kernel's threads gather the image operand.  NF <= 256;
 * `workspace` must hold hcConvF32TensorWorkspaceBytes(N, C, H, W, NF, HF, WF)
 * bytes of device memory, 1 KiB aligned (the split filters and the image as its
 * hi and lo parts: twice the size of x, channels rounded up to 32), and is
 * written by every call.  Fails on a device without tcgen05,
 * where hcMappedGemm computes the same convolution. */
HC_B200_API size_t hcConvF32TensorWorkspaceBytes(long long N, long long C, long long H,
                                                 long long W, long long NF, long long HF,
                                                 long long WF);
HC_B200_API int hcConvF32Tensor(HcContext c, const void *x, const void *f, void *out,
                                long long N, long long C, long long H, long long W,
                                long long NF, long long HF, long long WF, long long stride,
                                void *workspace, size_t workspaceBytes);

/* bf16 GEMM with fp32 accumulation on the tensor cores (tcgen05); falls back
 * to the bf16 tiled kernel for layouts TMA cannot describe (a pitch that is
 * not a multiple of 8 elements or a base that is not 16-byte aligned). */
HC_B200_API int hcGemmBf16(HcContext c, const void *a, const void *b, void *cOut,
                           long long M, long long N, long long K,
                           long long lda, long long ldb, long long ldc);

/* int8 weight-only dequant GEMM:
 *   out[m,n] = bf16( scale[n] * sum_k a[m,k] * float(w[k,n]) )
 * a bf16 [M,K], w int8 [K,N], scale fp32 [N], out bf16 [M,N].  `workspace`
 * must hold hcGemmW8A16WorkspaceBytes(N, K) bytes of device memory (the
 * weights converted to bf16); it is written by every call. */
HC_B200_API size_t hcGemmW8A16WorkspaceBytes(long long N, long long K);
/* What the form selected with the option `w8a16_variant` = 3 uses of the
 * workspace (its first bytes, 256-byte aligned): the weights are converted
 * inside the GEMM kernel, one band of 1024 columns at a time, into a ring of
 * three bands that the tiles read from L2 - 3 * K * 1024 * 2 bytes and a few
 * counters instead of the whole converted matrix.  The CTAs of that kernel wait
 * for one another (every CTA converts a share of every band), so its grid is
 * what the idle device holds at once: do not run it beside other kernels on
 * the same GPU - a CTA that cannot start makes the others' bounded waits run
 * out, and the call's result is then reported through hcKernelStatus (6 or 7). */
HC_B200_API size_t hcGemmW8A16BandedBytes(long long N, long long K);
HC_B200_API int hcGemmW8A16(HcContext c, const void *a, const void *w,
                            const float *scale, void *out, void *workspace,
                            size_t workspaceBytes, long long M, long long N,
                            long long K, long long lda, long long ldw,
                            long long ldc);

/* hcGemmW8A16 without a caller-provided workspace, for callers that must not
 * allocate device memory (a serving loop whose memory is handed out once at
 * start-up; a host that lends the library a stream but owns all allocations).
 * The converted weights go into a fixed scratch array built into the
 * library's device image instead, so roundUp(N,16) * K * 2 bytes must not
 * exceed hcGemmW8A16StaticMaxBytes() (32 MiB); larger problems are rejected
 * with an error that says so.  All calls on a device share that array: calls
 * ordered on one context are safe, calls whose GPU work overlaps race.  The
 * first call on a device resolves the array's address and loads the kernel
 * images; make it before starting any stream capture.  Later calls only look
 * up cached state and launch.
 * No counterpart in the reference: its runtime allocates with cuMemAlloc
 * whenever asked (gpu-runtime/cuda-runtime/src/Runtime.cpp:242-256) and has no
 * scratch-using kernels. */
HC_B200_API size_t hcGemmW8A16StaticMaxBytes(void);
HC_B200_API int hcGemmW8A16Static(HcContext c, const void *a, const void *w,
                                  const float *scale, void *out, long long M,
                                  long long N, long long K, long long lda,
                                  long long ldw, long long ldc);

/* ---- host buffers ------------------------------------------------------------
 * The row-wise workloads and the bf16 GEMM on matrices that live in HOST
 * memory: every pointer below is a host pointer.  The matrix is cut into row
 * chunks of about 16 MiB that stream through the GPU on three queues of the
 * context's device (upload of chunk i+1, kernel on chunk i, download of chunk
 * i-1 overlap; device slots are allocated on first use and kept by the
 * context), so a call costs little more than moving the data over the link
 * once each way.  Only whole rows reach the kernels: results are those of the
 * device entry points, bit for bit except that a row sum may differ in its last
 * bits when a chunk is short enough for hcReduceRows to take its other kernel.
 * A call returns when the result is in host memory.  The copies overlap only for page-locked memory: lock a range once
 * with hcHostPin (and release it with hcHostUnpin); pageable memory works but
 * serialises the three stages.  No counterpart in the reference, whose runtime
 * sees device pointers only and synchronises after every launch
 * (python/cpp/py-runtime/src/GpuRuntime.cpp:60-69). */
HC_B200_API int hcHostPin(HcContext c, void *ptr, size_t bytes);
HC_B200_API int hcHostUnpin(HcContext c, void *ptr);
HC_B200_API int hcSoftmaxRowsHost(HcContext c, const void *xHost, void *yHost,
                                  long long rows, long long cols, long long xPitch,
                                  long long yPitch, int dtype);
/* Either output may be NULL. */
HC_B200_API int hcReduceRowsHost(HcContext c, const void *xHost, void *sumHost,
                                 void *maxHost, long long rows, long long cols,
                                 long long pitch, int dtype);
/* c = a @ b in bf16 with fp32 accumulation: b [K, N] is uploaded whole, row
 * blocks of a [M, K] stream through, row blocks of c [M, N] come back. */
HC_B200_API int hcGemmBf16Host(HcContext c, const void *aHost, const void *bHost,
                               void *cHost, long long M, long long N, long long K,
                               long long lda, long long ldb, long long ldc);

/* Records `text` as the context's last error, reports it through the
 * context's callback and returns 1.  For code layered on this library. */
HC_B200_API int hcReportError(HcContext c, const char *text);

/* The conversion step alone: out[k,n] = bf16(w[k,n]). */
HC_B200_API int hcDequantW8(HcContext c, const void *w, void *out,
                            long long rows, long long cols, long long wPitch,
                            long long outPitch);

#ifdef __cplusplus
}
#endif
