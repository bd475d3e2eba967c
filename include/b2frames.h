/*
 * b2frames -- C ABI of the B200 post-decode frame path.
 *
 * One shared library, libb2frames.so, built for sm_100a.  Plain pointers and
 * sizes only; no C++ or torch types cross this boundary.  Each entry point names
 * the piece of facebookresearch/spdl it stands in for (path within that project).
 *
 * Conventions
 *   - Every function returns 0 on success.  On failure it returns a non-zero
 *     B2_ERR_* code and b2_last_error() gives a message for the calling thread.
 *     (The reference throws std::runtime_error from the same places; a binding
 *     turns the status into the host language's exception.)
 *   - Pointers named src/dst/base/descs are DEVICE pointers unless stated.
 *   - `stream` is a cudaStream_t passed as void*; 0x2 is the per-thread default
 *     stream (the reference's default, src/libspdl/cuda/types.h:32-39).
 *   - Work is enqueued on `stream` and the call returns without waiting unless
 *     the function says otherwise.  Inputs must stay alive until the stream has
 *     run past the call.
 *   - Re-entrant: no global mutable state a caller can observe; a call that takes
 *     `device` makes that device current for its duration and restores the caller's
 *     device.
 *   - No source or destination pointer, pitch, stride or width needs any alignment.
 *     The kernels read whole aligned segments, though: a source buffer must allow
 *     reads of every aligned 16-byte segment that holds at least one byte of it
 *     (b2_convert_resize) resp. every aligned 8-byte word (b2_convert_dense on rows
 *     that are not 16-byte aligned).  Any allocation that starts and ends on such
 *     boundaries -- cudaMalloc, every framework allocator -- satisfies this; a
 *     sub-allocation whose last bytes share a 16-byte segment with an unmapped page
 *     would not.  Nothing is ever written outside the destination elements.
 */
#ifndef B2FRAMES_H_
#define B2FRAMES_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2_ABI_VERSION 2

#if defined(__GNUC__)
#define B2_API __attribute__((visibility("default")))
#else
#define B2_API
#endif

enum b2_status {
  B2_OK = 0,
  B2_ERR_INVALID = 1, /* bad argument (shape, alignment of a required field, null pointer) */
  B2_ERR_CUDA = 2,    /* a CUDA runtime call failed; message holds the CUDA error name       */
  B2_ERR_LIMIT = 3    /* a size is beyond a stated maximum                                   */
};

/* B2_SRC_RGB_PLANAR / B2_SRC_RGB_INTERLEAVED: already-decoded 8-bit RGB as a JPEG decoder emits
 * it (src/libspdl/cuda/nvjpeg/decoding.cpp:56-95); accepted by b2_convert_resize only. */
enum b2_src_format {
  B2_SRC_NV12 = 0,
  B2_SRC_I420 = 1,
  B2_SRC_RGB_PLANAR = 2,
  B2_SRC_RGB_INTERLEAVED = 3
};
enum b2_layout { B2_NCHW = 0, B2_NHWC = 1 };
enum b2_dtype { B2_U8 = 0, B2_F32 = 1, B2_BF16 = 2 };
enum b2_order { B2_RGB = 0, B2_BGR = 1 };
/* Which arithmetic turns (Y,U,V) into 8-bit RGB.
 *   B2_ARITH_REFERENCE  the reference's CUDA kernel: fp32 matrix product, truncation
 *                       (src/libspdl/cuda/detail/color_conversion.cu:20-86).  The default.
 *   B2_ARITH_SWSCALE    the reference's CPU route: the integer arithmetic of libswscale's
 *                       unscaled yuv420p -> rgb24 converter, which the filter graph built by
 *                       src/libspdl/core/detail/ffmpeg/filter_graph.cpp:50-65 from
 *                       "format=pix_fmts=rgb24" (src/spdl/io/_preprocessing.py:250-251) ends in.
 *                       matrix_coeff is then the colourspace number sws_getCoefficients() takes
 *                       (1 BT.709, 4 FCC, 5/6 BT.601, 7 SMPTE 240M, 9/10 BT.2020, anything else
 *                       BT.601) and full_range its srcRange. */
enum b2_arith { B2_ARITH_REFERENCE = 0, B2_ARITH_SWSCALE = 1 };

/* Message for the last failure on the calling thread ("" if none). */
B2_API const char* b2_last_error(void);
B2_API int b2_abi_version(void);

/* Create/attach the primary context of `device`.
 * Replaces spdl::cuda::init_cuda (src/libspdl/cuda/utils.cpp:25-37). */
B2_API int b2_init(int device);
B2_API int b2_device_count(int* count);

/* Wait for `stream` on `device`.
 * Replaces spdl::cuda::synchronize_stream (src/libspdl/cuda/utils.cpp:39-43). */
B2_API int b2_stream_synchronize(int device, void* stream);

/* ------------------------------------------------------------------------------------------
 * Colour conversion, reference signature.
 *
 * Drop-in for spdl::cuda::detail::nv12_to_planar_rgb / nv12_to_planar_bgr
 * (src/libspdl/cuda/detail/color_conversion.cu:155-193; the function-pointer type
 * Nv2Converter at src/libspdl/cuda/color_conversion.cpp:24-25).  Same argument
 * order and meaning: `src` holds num_frames packed NV12 frames of
 * (height + height/2) rows, rows `src_pitch` bytes apart, frames
 * (height + height/2) * width bytes apart; `dst` receives planar u8
 * [num_frames, 3, height, width], rows `dst_pitch` apart, planes
 * height * dst_pitch apart, frames 3 * height * width apart.
 * matrix_coefficients outside 1..10 means 1 (BT.709).  Runs on the current device.
 * A trailing odd column or row is left untouched, as in the reference.
 * ---------------------------------------------------------------------------------------- */
B2_API int b2_nv12_to_planar_rgb(void* stream, const uint8_t* src, int src_pitch, uint8_t* dst,
                          int dst_pitch, int width, int height, int num_frames,
                          int matrix_coefficients);
B2_API int b2_nv12_to_planar_bgr(void* stream, const uint8_t* src, int src_pitch, uint8_t* dst,
                          int dst_pitch, int width, int height, int num_frames,
                          int matrix_coefficients);

/* ------------------------------------------------------------------------------------------
 * Colour conversion, general form (same arithmetic, more layouts).
 *
 * Covers what the reference does in separate passes around its kernel: the
 * planar->interleaved permute and the float()/255, (x-mean)/std, .to(bf16) that
 * user code applies afterwards (examples/imagenet_classification.py:95-106), and
 * planar-chroma (I420) input as produced by convert_frames for yuv420p
 * (src/libspdl/core/detail/ffmpeg/conversion.cpp:218-260).
 *
 * out[slot] = value(channel(slot)) * scale[slot] + bias[slot] for float outputs
 * (one fused multiply-add in fp32; bf16 rounds that to nearest even); u8 outputs
 * ignore scale/bias.  slot order is R,G,B or B,G,R per `order`.
 * ---------------------------------------------------------------------------------------- */
typedef struct b2_dense_args {
  uint32_t struct_size;     /* sizeof(b2_dense_args), for forward compatibility            */
  int32_t device;
  const void* y;            /* luma of frame 0                                              */
  const void* u;            /* NV12: interleaved UV plane of frame 0; I420: U plane         */
  const void* v;            /* I420: V plane; NV12: ignored                                 */
  /* Optional pointer table (device memory, num_frames entries each) for frames that do not
   * sit at a fixed stride, e.g. decoder surfaces.  When y_table is non-null the kernel takes
   * frame i's planes from y_table[i], u_table[i] (and v_table[i]) and ignores y/u/v and the
   * frame strides. */
  const void* const* y_table;
  const void* const* u_table;
  const void* const* v_table;
  int64_t y_pitch, uv_pitch;              /* bytes between rows                             */
  int64_t y_frame_stride, uv_frame_stride; /* bytes between frames                          */
  int32_t src_format;       /* b2_src_format                                                */
  int32_t width, height, num_frames;
  int32_t matrix_coeff;     /* 1..10, else 1                                                */
  int32_t full_range;       /* 0: limited range (the reference); 1: full range, no offset   */
  void* dst;
  int64_t dst_frame_stride; /* elements between frames; 0 = packed (3*height*width)         */
  int32_t layout, dtype, order;
  float scale[3], bias[3];
  int32_t reserved0;        /* tail padding of the version-1 struct; ignored                */
  /* --- fields of ABI version 2: a caller whose struct_size is that of version 1 (168) gets
   *     zeros for them --- */
  int32_t arith;            /* b2_arith                                                      */
  int32_t reserved1;
} b2_dense_args;

B2_API int b2_convert_dense(const b2_dense_args* args, void* stream);

/* ------------------------------------------------------------------------------------------
 * Fused convert -> bilinear resize -> crop -> scale/bias over a ragged batch.
 *
 * Stands in for the resize that follows decode in the reference -- NPP resize
 * (src/libspdl/cuda/npp/detail/resize.cpp:37-116), the NVDEC crop/scale
 * parameters (src/libspdl/cuda/nvdec/detail/utils.cpp:133-220) and the
 * scale/crop filter strings (src/spdl/io/_preprocessing.py:122-254) -- fused
 * with the colour conversion above and the normalise of user code.  Filter:
 * bilinear, half-pixel centres, no antialias.  Each image has a descriptor; all
 * images write an out_h x out_w result.
 * ---------------------------------------------------------------------------------------- */
/* Planes per source format: NV12 = Y, interleaved UV (v_off unused); I420 = Y, U, V;
 * RGB planar = three full-size planes in y_off, u_off, v_off (y_pitch for the first, uv_pitch
 * for the other two); RGB interleaved = one plane of 3-byte pixels in y_off / y_pitch. */
typedef struct b2_image_desc {
  uint64_t y_off, u_off, v_off; /* byte offsets of the planes from `base`                   */
  int32_t y_pitch, uv_pitch;
  int32_t src_w, src_h;
  int32_t crop_x, crop_y;       /* where output (0,0) sits in the resized grid; negative when
                                 * the resized image is smaller than the output (letterbox)  */
  float scale_x, scale_y;       /* source size / resized size                               */
  int32_t resized_w, resized_h; /* size of the resized grid; output pixels that fall outside
                                 * it take args->pad_value.  0 = unbounded (version 1: these
                                 * were reserved zeros), every output pixel maps into the
                                 * image with edge clamping                                  */
} b2_image_desc;                /* 64 bytes */

typedef struct b2_resize_args {
  uint32_t struct_size;
  int32_t device;
  const void* base;             /* device buffer holding every image                        */
  const b2_image_desc* descs;   /* device table, num_images entries                         */
  int32_t num_images, src_format;
  int32_t out_w, out_h;
  int32_t matrix_coeff, full_range;
  int32_t layout, dtype, order;
  int32_t max_src_w;            /* largest src_w in the table (sizes the staging tile)      */
  void* dst;
  int64_t dst_image_stride;     /* elements; 0 = packed                                     */
  float scale[3], bias[3];
  /* --- fields of ABI version 2: a caller whose struct_size is that of version 1 (104) gets
   *     zeros for them --- */
  int32_t arith;                /* b2_arith (YUV sources)                                   */
  /* Clip stacking.  With frames_per_group = T > 1, image i is frame t = i % T of group
   * g = i / T and starts at element g * dst_group_stride + t * dst_image_stride; with
   * dst_plane_stride (NCHW: elements between the colour planes of one image; 0 = out_h*out_w)
   * this writes the [N, C, T, H, W] layout of examples/video_classification/utils/pipeline.py:137
   * directly (image stride H*W, plane stride T*H*W, group stride 3*T*H*W). */
  int32_t frames_per_group;
  int64_t dst_plane_stride;
  int64_t dst_group_stride;
  /* Letterbox colour as R, G, B on the 0..255 scale, for output pixels outside an image's
   * resized grid (see b2_image_desc.resized_w); it passes through the same rounding /
   * scale / bias as every other pixel.  The reference pads with a colour name
   * (src/spdl/io/_preprocessing.py:220-223), black by default. */
  float pad_value[3];
  int32_t debug_flags;          /* B2_DEBUG_*; 0 in production                               */
  /* Optional device word (may be null).  The kernel ORs B2_STATUS_* bits into it when it leaves
   * an image or a tile of output rows unwritten; the caller clears it before the call and reads
   * it after the stream has run.  The call itself still returns B2_OK: the host cannot see the
   * descriptor table, which lives in device memory. */
  int32_t* status;
  /* Row-sparse sources (optional; one pair of maps for the whole call, so for batches whose
   * images share one geometry, e.g. video frames).  A caller that uploads only the source rows a
   * geometry touches stores them back to back and says where each row went: with luma_row_map
   * non-null, row r of the first plane (of every plane for RGB sources) is read from row
   * luma_row_map[r] of the plane the descriptor points to, and row r of the half-height planes of
   * a YUV source from row chroma_row_map[r].  Device arrays of int32; entries of rows the geometry
   * does not touch are never read.  b2_touched_rows computes the maps.  The reference uploads
   * whole frames (src/libspdl/cuda/transfer.cpp:37-66); a 4K frame resized to 224x224 touches a
   * quarter of its rows. */
  const int32_t* luma_row_map;
  const int32_t* chroma_row_map;
} b2_resize_args;

enum b2_resize_status_bits {
  B2_STATUS_IMAGE_TOO_WIDE = 1, /* a descriptor needs more staging than max_src_w provides:
                                 * the image was skipped                                     */
  B2_STATUS_WAIT_EXPIRED = 2,   /* a bounded wait for staged rows ran out: the tile was skipped */
  B2_STATUS_BAD_GEOMETRY = 4    /* src_w/src_h < 1, a non-positive / non-finite scale or source
                                 * coordinates beyond 2^22: skipped; or a row map that marks a
                                 * row the geometry reads as absent (row 0 is read instead)   */
};
/* B2_DEBUG_EXPIRE_WAIT: after its rows have arrived, every tile also waits (bounded, a few
 * polls) on a barrier that nothing completes, so that the give-up path can be tested without
 * any copy in flight.  Outputs stay untouched and B2_STATUS_WAIT_EXPIRED is reported. */
enum b2_debug_flags { B2_DEBUG_EXPIRE_WAIT = 1 };

B2_API int b2_convert_resize(const b2_resize_args* args, void* stream);

/* Host helper (no CUDA call): the source rows that the vertical geometry of `desc` touches when
 * out_h output rows are produced, computed with the arithmetic of the kernel.  luma_map receives
 * desc->src_h entries, chroma_map (YUV source formats only, may be null otherwise)
 * (desc->src_h + 1) / 2: the index of the row among the touched rows of its plane, in order, or -1
 * for a row that is never read.  n_luma / n_chroma receive the numbers of touched rows.  Together
 * with b2_resize_args.luma_row_map this lets a caller upload a fraction of each frame.  No
 * counterpart in the reference. */
B2_API int b2_touched_rows(const b2_image_desc* desc, int src_format, int out_h, int32_t* luma_map,
                    int32_t* chroma_map, int32_t* n_luma, int32_t* n_chroma);

/* Host helper (no CUDA call): packs selected rows of a batch of equally laid out HOST planes.
 * For every frame f < num_frames and i < num_rows, row_bytes bytes are copied from
 * src + f * src_frame_stride + rows[i] * src_pitch to dst + f * dst_frame_stride + i * row_bytes.
 * It takes the place of the whole-frame copy with which the reference batches decoded frames
 * (src/libspdl/core/detail/ffmpeg/conversion.cpp:171-216) when only the touched rows are to be
 * uploaded; dst is typically page-locked.  With num_rows = 1, rows = {0} and row_bytes = the
 * frame size it is the whole-frame staging copy.  Batches of several MiB are cut into ranges for
 * several host threads (B2_HOST_COPY_THREADS; default half the hardware threads, at most 8), and
 * consecutive rows of a tightly pitched source go as one memcpy. */
B2_API int b2_copy_rows(void* dst, int64_t dst_frame_stride, const void* src, int64_t src_frame_stride,
                 int64_t src_pitch, const int32_t* rows, int num_rows, int64_t row_bytes,
                 int num_frames);

/* Host helper (no CUDA call): memcpy of nbytes, cut into slices for several host threads when it
 * is several MiB long (same thread count as b2_copy_rows).  Like b2_copy_rows and b2_pack_host
 * it writes with streaming stores: it is the staging copy of host data into page-locked memory,
 * which the copy engine reads next, and an upload right after a cached copy runs at half the
 * link's rate.  The reference pins such arrays with Tensor.pin_memory() in
 * spdl.io.transfer_tensor (src/spdl/io/_transfer.py:84). */
B2_API int b2_copy_host(void* dst, const void* src, size_t nbytes);

/* Host helper (no CUDA call): packs num_items host arrays of different sizes into one buffer,
 * item i (sizes[i] bytes at srcs[i]) to dst + dst_offsets[i]; whole items are dealt out to several
 * host threads when the batch is several MiB long.  The staging copy of a list of decoded
 * images of different sizes, which the reference cannot batch at all (its convert_frames wants
 * equal sizes, src/libspdl/core/detail/ffmpeg/conversion.cpp:307-390, so such images are
 * resized one by one on the CPU first: load_image_batch, src/spdl/io/_composite.py:438-463). */
B2_API int b2_pack_host(void* dst, const void* const* srcs, const int64_t* sizes,
                 const int64_t* dst_offsets, int num_items);

/* ------------------------------------------------------------------------------------------
 * Frame batching.
 *
 * Replaces FrameBuffer::push (src/libspdl/cuda/nvdec/detail/buffer.cpp:31-74): copies
 * `num_frames` pitched NV12 surfaces (device pointer table + pitch table, both in device
 * memory) into one packed [num_frames, height*3/2, width] batch in a single launch, without
 * the per-frame stream synchronisation.
 * ---------------------------------------------------------------------------------------- */
B2_API int b2_gather_surfaces(const void* const* surfaces, const int64_t* pitches, int num_frames,
                       int width, int height, uint8_t* dst, int device, void* stream);

/* ------------------------------------------------------------------------------------------
 * Buffer transfer and storage.
 *
 * b2_transfer_h2d replaces transfer_buffer_impl (src/libspdl/cuda/transfer.cpp:37-66):
 * pinned source -> asynchronous copy on `stream` followed by a stream synchronise;
 * pageable source -> blocking copy.  b2_transfer_h2d_async is the same copy without the
 * wait, for callers that overlap transfers.  b2_transfer_d2h replaces the device->host
 * overload (src/libspdl/cuda/transfer.cpp:91-118): blocking.
 * b2_alloc_pinned / b2_free_pinned replace alloc_pinned / dealloc_pinned
 * (src/libspdl/cuda/storage.cpp:22-38); b2_device_alloc / b2_device_free are the default
 * allocator of CUDAStorage (src/libspdl/cuda/storage.cpp:44-58).
 * ---------------------------------------------------------------------------------------- */
B2_API int b2_transfer_h2d(void* dst, const void* host_src, size_t nbytes, int src_is_pinned, int device,
                    void* stream);
B2_API int b2_transfer_h2d_async(void* dst, const void* host_src, size_t nbytes, int device,
                          void* stream);
/* The pageable branch of transfer_buffer_impl (src/libspdl/cuda/transfer.cpp:59-63: a blocking
 * cudaMemcpy, which the driver stages on one thread at about a fifth of the link's rate) through
 * the CALLER's page-locked staging buffer instead: the buffer is cut into two halves, the staging
 * copy of one half (b2_copy_host, several host threads) overlaps the asynchronous upload of the
 * other on `stream`.  Returns when all the data is on the device, like b2_transfer_h2d.
 * staging_bytes >= 512; a few tens of MiB are enough. */
B2_API int b2_transfer_h2d_staged(void* dst, const void* host_src, size_t nbytes, void* staging,
                           size_t staging_bytes, int device, void* stream);
B2_API int b2_transfer_d2h(void* host_dst, const void* src, size_t nbytes, int device);
/* b2_transfer_d2h for a large pageable destination, through the CALLER's page-locked staging
 * buffer cut into two halves: the download of one half on `stream` overlaps the copy of the other
 * half out to host_dst (b2_copy_host, several host threads).  Returns when host_dst is complete.
 * The reference's device->host transfer (src/libspdl/cuda/transfer.cpp:91-118) is one blocking
 * cudaMemcpy into pageable memory. */
B2_API int b2_transfer_d2h_staged(void* host_dst, const void* src, size_t nbytes, void* staging,
                           size_t staging_bytes, int device, void* stream);
B2_API int b2_alloc_pinned(void** host_ptr, size_t nbytes);
B2_API int b2_free_pinned(void* host_ptr);
B2_API int b2_device_alloc(void** ptr, size_t nbytes, int device);
B2_API int b2_device_free(void* ptr, int device);

/* Per-frame checksum of a packed byte batch: out[i] = sum over j of
 * (byte[i][j] + 1) * (1 + j mod 65521), as uint64.  `out` is device memory,
 * num_frames entries, overwritten.  No counterpart in the reference; used to
 * verify full-size results without copying them back. */
B2_API int b2_frame_checksum(const uint8_t* src, int64_t frame_bytes, int num_frames, uint64_t* out,
                      int device, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B2FRAMES_H_ */
