// C entry points over the reference's OWN CUDA kernels, for the test-suite only.
//
// TEST INFRASTRUCTURE (see oracle/__init__.py): this file is compiled together with the
// reference's unmodified sources (energonai/kernel/cuda_native/csrc/scale_mask_softmax_kernel.cu,
// transpose_pad_fusion_kernel.cu, layer_norm_cuda_kernel.cu), taken from the reference checkout
// where it lies, into oracle/_ref/libenergon_ref.so by oracle/ref_cuda/build_ref.py.  It declares
// the launchers those files define (their prototypes are the interface the reference's own
// pybind wrappers use: scale_mask_softmax_wrapper.cpp:7-12, transpose_pad_fusion_wrapper.cpp,
// layer_norm_cuda.cpp:60-73) and forwards raw pointers to them.  The library is the second
// oracle for the kernels the reference has no test for, and the same-GPU baseline they are timed
// against.  Nothing in the product links, loads or imports it.
#include <ATen/ATen.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

// ---- prototypes of the reference's launchers (definitions live in its .cu files) -------------
template <typename T>
void ker_scale_mask_softmax_launcher(int batch_size, int batch_seq_len, int head_num, T *correlation,
                                     const int *real_seq_len);
template <typename T>
void transpose_depad(const T *src, const int batch_size, const int seq_len, const int *seq_lens, const int head_num,
                     const int size_per_head, T *dst);
template <typename T>
void transpose_pad(const T *src, const int batch_size, const int seq_len, const int *seq_lens, const int head_num,
                   const int size_per_head, T *dst);
void build_sequence_length_padding_offset_kernelLauncher(const int *sequence_length, const int batch_size,
                                                         const int max_seq_len, int *valid_word_num, int *tmp_mask_offset);
template <typename T>
void remove_sequence_length_padding_kernelLauncher(const T *src, T *tgt, const int *tmp_mask_offset, int *mask_offset,
                                                   const int m, const int n);
template <typename T>
void rebuild_sequence_length_padding_kernelLauncher(const T *src, T *tgt, const int *mask_offset, const int m, const int n);
template <typename T>
void transpose_rebuild_padding_kernelLauncher(T *Q, T *K, T *V, T *q_buf, T *k_buf, T *v_buf, const int batch_size,
                                              const int seq_len, const int head_num, const int size_per_head,
                                              const int valid_word_num, const int *mask_offset);
template <typename T>
void transpose_remove_padding_kernelLauncher(T *src, T *dst, const int valid_word_num, const int batch_size,
                                             const int seq_len, const int head_num, const int size_per_head,
                                             const int *mask_offset);
void cuda_layer_norm(at::Tensor *output, at::Tensor *mean, at::Tensor *invvar, at::Tensor *input, int n1, int n2,
                     at::IntArrayRef normalized_shape, at::Tensor *gamma, at::Tensor *beta, double epsilon);

#define REF_API extern "C" __attribute__((visibility("default")))

static int last_error() { return cudaGetLastError() == cudaSuccess ? 0 : -1; }

// dtype: 0 fp32, 1 fp16 (the two the reference instantiates); all launches go to the default
// stream, as in the reference.
REF_API int ref_scale_mask_softmax(int batch, int seq_len, int heads, void *scores, const int *real_len, int dtype) {
  if (dtype == 0) ker_scale_mask_softmax_launcher<float>(batch, seq_len, heads, (float *)scores, real_len);
  else ker_scale_mask_softmax_launcher<__half>(batch, seq_len, heads, (__half *)scores, real_len);
  return last_error();
}
REF_API int ref_transpose_pad(const void *src, int batch, int seq_len, const int *lens, int heads, int d, void *dst, int dtype) {
  if (dtype == 0) transpose_pad<float>((const float *)src, batch, seq_len, lens, heads, d, (float *)dst);
  else transpose_pad<half>((const half *)src, batch, seq_len, lens, heads, d, (half *)dst);
  return last_error();
}
REF_API int ref_transpose_depad(const void *src, int batch, int seq_len, const int *lens, int heads, int d, void *dst, int dtype) {
  if (dtype == 0) transpose_depad<float>((const float *)src, batch, seq_len, lens, heads, d, (float *)dst);
  else transpose_depad<half>((const half *)src, batch, seq_len, lens, heads, d, (half *)dst);
  return last_error();
}
REF_API int ref_build_padding_offsets(const int *lens, int batch, int seq_len, int *valid_word_num, int *tmp_mask_offset) {
  build_sequence_length_padding_offset_kernelLauncher(lens, batch, seq_len, valid_word_num, tmp_mask_offset);
  return last_error();
}
REF_API int ref_remove_padding(const void *src, void *tgt, const int *tmp_off, int *off, int m, int n, int dtype) {
  if (dtype == 0) remove_sequence_length_padding_kernelLauncher<float>((const float *)src, (float *)tgt, tmp_off, off, m, n);
  else remove_sequence_length_padding_kernelLauncher<half>((const half *)src, (half *)tgt, tmp_off, off, m, n);
  return last_error();
}
REF_API int ref_rebuild_padding(const void *src, void *tgt, const int *off, int m, int n, int dtype) {
  if (dtype == 0) rebuild_sequence_length_padding_kernelLauncher<float>((const float *)src, (float *)tgt, off, m, n);
  else rebuild_sequence_length_padding_kernelLauncher<half>((const half *)src, (half *)tgt, off, m, n);
  return last_error();
}
REF_API int ref_transpose_rebuild_padding(void *Q, void *K, void *V, void *q, void *k, void *v, int batch, int seq_len,
                                          int heads, int d, int valid, const int *off, int dtype) {
  if (dtype == 0)
    transpose_rebuild_padding_kernelLauncher<float>((float *)Q, (float *)K, (float *)V, (float *)q, (float *)k, (float *)v,
                                                    batch, seq_len, heads, d, valid, off);
  else
    transpose_rebuild_padding_kernelLauncher<half>((half *)Q, (half *)K, (half *)V, (half *)q, (half *)k, (half *)v, batch,
                                                   seq_len, heads, d, valid, off);
  return last_error();
}
REF_API int ref_transpose_remove_padding(void *src, void *dst, int valid, int batch, int seq_len, int heads, int d,
                                         const int *off, int dtype) {
  if (dtype == 0) transpose_remove_padding_kernelLauncher<float>((float *)src, (float *)dst, valid, batch, seq_len, heads, d, off);
  else transpose_remove_padding_kernelLauncher<half>((half *)src, (half *)dst, valid, batch, seq_len, heads, d, off);
  return last_error();
}

// forward_affine of the reference (layer_norm_cuda.cpp:82-103) on raw pointers: x, y [n1, n2] in
// `dtype` (0 fp32, 1 fp16, 2 bf16), gamma / beta [n2] in the same type, mean / invvar fp32 [n1].
REF_API int ref_layer_norm(void *y, float *mean, float *invvar, const void *x, const void *gamma, const void *beta,
                           long long n1, int n2, double eps, int dtype) {
  const auto st = dtype == 0 ? at::kFloat : dtype == 1 ? at::kHalf : at::kBFloat16;
  const auto opt = at::TensorOptions().dtype(st).device(at::kCUDA);
  const auto optf = at::TensorOptions().dtype(at::kFloat).device(at::kCUDA);
  at::Tensor in = at::from_blob(const_cast<void *>(x), {n1, n2}, opt), out = at::from_blob(y, {n1, n2}, opt);
  at::Tensor g = at::from_blob(const_cast<void *>(gamma), {n2}, opt), b = at::from_blob(const_cast<void *>(beta), {n2}, opt);
  at::Tensor mu = at::from_blob(mean, {n1}, optf), iv = at::from_blob(invvar, {n1}, optf);
  const int64_t shape[1] = {n2};
  cuda_layer_norm(&out, &mu, &iv, &in, (int)n1, n2, at::IntArrayRef(shape, 1), &g, &b, eps);
  return last_error();
}
