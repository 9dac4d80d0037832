// aten kernels the device core itself provides for `spyre` tensors: allocation,
// metadata views and the host<->device copy with its stick relayout.  Same
// registrations as the reference (torch_spyre/csrc/spyre_mem.cpp:557-711); the
// copy calls the relayout entry points of the kernel library where the reference
// built a SenDataConvert + DMA graph (spyre_mem.cpp:281-438).
#include <ATen/ATen.h>
#include <ATen/native/Resize.h>
#include <ATen/native/TensorShape.h>
#include <ATen/ops/_copy_from_native.h>
#include <ATen/ops/as_strided_cpu_dispatch.h>
#include <ATen/ops/set_cpu_dispatch.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <algorithm>
#include <numeric>

#include "../../../include/spyre_b200.h"
#include "spyre_storage.h"

namespace spyre {
namespace {

void check_status(int rc, const char* what) {
  TORCH_CHECK(rc == TS_OK, what, ": ", ts_status_string(rc), " (", rc, ") ", ts_last_cuda_error());
}

int checked_elem_bytes(c10::ScalarType t) {
  const int eb = (int)c10::elementSize(t);
  TORCH_CHECK(eb == 1 || eb == 2 || eb == 4 || eb == 8, "spyre tensors hold 1-, 2-, 4- or 8-byte elements; got ",
              t);
  return eb;
}

// Row-major base shape a (size, stride) pair is a view of: the sizes in decreasing-
// stride order when the strides describe a dense permutation, otherwise the flat span.
std::vector<int64_t> base_shape_for(c10::IntArrayRef size, c10::IntArrayRef stride) {
  if (size.empty()) return {1};
  std::vector<int64_t> shape(size.begin(), size.end());
  std::vector<size_t> order(size.size());
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(),
                   [&](size_t a, size_t b) { return stride[a] > stride[b]; });
  int64_t expect = 1;
  bool dense = true;
  for (auto it = order.rbegin(); it != order.rend(); ++it) {
    if (size[*it] != 1 && stride[*it] != expect) dense = false;
    expect *= size[*it];
  }
  if (dense) {
    std::vector<int64_t> base;
    for (size_t d : order) base.push_back(size[d]);
    return base;
  }
  int64_t span = 1;
  for (size_t d = 0; d < size.size(); ++d) {
    if (size[d] == 0) return {0};
    span += (size[d] - 1) * stride[d];
  }
  return {span};
}

at::Tensor make_tensor(std::vector<int64_t> base, c10::IntArrayRef size, c10::IntArrayRef stride,
                       c10::ScalarType scalar_type, c10::Device device) {
  const int eb = checked_elem_bytes(scalar_type);
  int64_t numel = 1;
  for (auto s : base) numel *= s;
  const int64_t nbytes = numel == 0 ? 0 : stick_nbytes(base, eb);
  const c10::cuda::CUDAGuard guard(device.index());
  auto storage_impl = c10::make_intrusive<c10::StorageImpl>(
      c10::StorageImpl::use_byte_size_t(), nbytes, spyre_allocator(), /*resizable=*/false);
  auto* ctx = static_cast<StorageCtx*>(storage_impl->data_ptr().get_context());
  ctx->elem_bytes = eb;
  ctx->base_shape = std::move(base);
  constexpr c10::DispatchKeySet ks(c10::DispatchKey::PrivateUse1);
  auto tensor = at::detail::make_tensor<c10::TensorImpl>(c10::Storage(storage_impl), ks,
                                                         c10::scalarTypeToTypeMeta(scalar_type));
  tensor.unsafeGetTensorImpl()->set_sizes_and_strides(size, stride);
  return tensor;
}

c10::Device resolve_device(std::optional<c10::Device> device_opt) {
  c10::Device d = device_opt.value_or(c10::Device(c10::DeviceType::PrivateUse1, -1));
  TORCH_CHECK(d.is_privateuseone());
  if (d.index() < 0) d = c10::Device(c10::DeviceType::PrivateUse1, c10::cuda::current_device());
  return d;
}

at::Tensor spyre_empty(c10::IntArrayRef size, std::optional<c10::ScalarType> dtype_opt,
                       std::optional<c10::Layout> layout_opt, std::optional<c10::Device> device_opt,
                       std::optional<bool> pin_memory_opt,
                       std::optional<c10::MemoryFormat> memory_format_opt) {
  TORCH_CHECK(c10::layout_or_default(layout_opt) == c10::Layout::Strided,
              "Non strided layout not supported");
  TORCH_CHECK(!c10::pinned_memory_or_default(pin_memory_opt), "Pin memory can only be on CPU");
  at::detail::check_size_nonnegative(size);
  const auto dtype = c10::dtype_or_default(dtype_opt);
  // A 0-dim tensor is a 1-element 1-D tensor on the device (spyre_mem.cpp:625-631).
  std::vector<int64_t> shape(size.begin(), size.end());
  if (shape.empty()) shape = {1};
  std::vector<int64_t> strides(shape.size());
  int64_t s = 1;
  for (int i = (int)shape.size() - 1; i >= 0; --i) {
    strides[i] = s;
    s *= std::max<int64_t>(shape[i], 1);
  }
  return make_tensor(shape, shape, strides, dtype, resolve_device(device_opt));
}

at::Tensor spyre_empty_strided(c10::IntArrayRef size, c10::IntArrayRef stride,
                               std::optional<c10::ScalarType> dtype_opt,
                               std::optional<c10::Layout> layout_opt,
                               std::optional<c10::Device> device_opt,
                               std::optional<bool> pin_memory_opt) {
  at::detail::check_size_nonnegative(size);
  const auto dtype = c10::dtype_or_default(dtype_opt);
  if (size.empty()) return make_tensor({1}, {1}, {1}, dtype, resolve_device(device_opt));
  return make_tensor(base_shape_for(size, stride), size, stride, dtype, resolve_device(device_opt));
}

at::Tensor spyre_as_strided(const at::Tensor& self, c10::IntArrayRef size, c10::IntArrayRef stride,
                            std::optional<int64_t> storage_offset) {
  // metadata only (spyre_mem.cpp:641-646)
  return at::cpu::as_strided(self, size, stride, storage_offset);
}

at::Tensor& spyre_set_storage(at::Tensor& result, at::Storage storage, int64_t storage_offset,
                              c10::IntArrayRef size, c10::IntArrayRef stride) {
  return at::cpu::set_(result, std::move(storage), storage_offset, size, stride);
}

at::Tensor spyre_view(const at::Tensor& self, c10::SymIntArrayRef size) {
  return at::native::view(self, C10_AS_INTARRAYREF_SLOW(size));
}

at::Tensor spyre_reshape_alias(const at::Tensor& self, c10::IntArrayRef size, c10::IntArrayRef stride) {
  return at::native::_reshape_alias(self, size, stride);
}

// ---- copies --------------------------------------------------------------------------

struct LayoutArrays {
  int64_t dsize[TS_MAX_DIMS], dstride[TS_MAX_DIMS];
  int32_t dmap[TS_MAX_DIMS];
  int ndev;
};
LayoutArrays layout_of(c10::IntArrayRef shape, int elem_bytes) {
  LayoutArrays l;
  std::vector<int64_t> s(shape.begin(), shape.end());
  if (s.empty()) s = {1};
  l.ndev = ts_layout_init(s.data(), (int)s.size(), elem_bytes, nullptr, l.dsize, l.dstride, l.dmap);
  TORCH_CHECK(l.ndev > 0, "tensor rank not supported by the stick layout: ", s.size());
  return l;
}

cudaStream_t current_stream(c10::DeviceIndex dev) { return c10::cuda::getCurrentCUDAStream(dev); }

// CUDA tensor holding the row-major base of a spyre tensor's storage (a temporary).
at::Tensor base_to_rowmajor(const at::Tensor& t) {
  StorageCtx* ctx = storage_ctx(t);
  auto opts = at::TensorOptions().dtype(t.scalar_type()).device(at::Device(at::kCUDA, ctx->device));
  at::Tensor raw = at::empty(ctx->base_shape, opts);
  if (raw.numel() == 0) return raw;
  const auto lay = layout_of(ctx->base_shape, ctx->elem_bytes);
  auto strides = raw.strides().vec();
  check_status(ts_relayout_from_sticks(ctx->ptr, raw.data_ptr(), ctx->elem_bytes,
                                       ctx->base_shape.data(), strides.data(),
                                       (int)ctx->base_shape.size(), lay.dsize, lay.dstride, lay.dmap,
                                       lay.ndev, current_stream(ctx->device)),
               "relayout from sticks");
  return raw;
}
void rowmajor_to_base(const at::Tensor& raw, const at::Tensor& t) {
  StorageCtx* ctx = storage_ctx(t);
  if (raw.numel() == 0) return;
  const auto lay = layout_of(ctx->base_shape, ctx->elem_bytes);
  auto strides = raw.strides().vec();
  check_status(ts_relayout_to_sticks(raw.data_ptr(), ctx->ptr, ctx->elem_bytes, ctx->base_shape.data(),
                                     strides.data(), (int)ctx->base_shape.size(), lay.dsize,
                                     lay.dstride, lay.dmap, lay.ndev, current_stream(ctx->device)),
               "relayout to sticks");
}
// The spyre tensor `t` as a strided view into a row-major CUDA copy of its base.
at::Tensor view_in(const at::Tensor& raw, const at::Tensor& t) {
  return raw.view({-1}).as_strided(t.sizes(), t.strides(), t.storage_offset());
}

// `non_blocking` is honoured for a pinned source, as torch's own CUDA copies do: the copies and
// relayout kernels are queued on the current stream and the call returns; the caller keeps the
// host buffer unchanged until the stream has passed that point.  (The staging block goes back to
// the caching allocator at once: it is bound to the current stream, and every copy into it is
// followed on that stream by the relayout kernel that consumes it, so later work on the stream
// cannot see it early.)
void host_to_device(const at::Tensor& src_cpu, const at::Tensor& dst, bool non_blocking) {
  StorageCtx* ctx = storage_ctx(dst);
  const c10::cuda::CUDAGuard guard(ctx->device);
  at::Tensor src = src_cpu.dim() == 0 && dst.dim() == 1 ? src_cpu.reshape({1}) : src_cpu;
  if (src.sizes() != dst.sizes()) src = src.expand(dst.sizes());
  if (dst.numel() == 0) return;
  cudaStream_t st = current_stream(ctx->device);
  if (is_canonical(dst)) {
    auto shape = dst.sizes().vec();
    if (shape.empty()) shape = {1};
    auto strides = src.strides().vec();
    if (strides.empty()) strides = {1};
    for (auto s : strides) TORCH_CHECK(s >= 0, "negative host strides are not supported");
    // chunks of the host span go through a small staging block, copy and relayout overlapped
    const int64_t want = std::max<int64_t>(
        ts_copy_staging_bytes(ctx->elem_bytes, shape.data(), strides.data(), (int)shape.size()), 256);
    void* staging = c10::cuda::CUDACachingAllocator::raw_alloc_with_stream(want, st);
    const auto lay = layout_of(shape, ctx->elem_bytes);
    int rc = ts_copy_host_to_sticks_pipelined(src.data_ptr(), staging, want, ctx->ptr, ctx->elem_bytes,
                                              shape.data(), strides.data(), (int)shape.size(), lay.dsize,
                                              lay.dstride, lay.dmap, lay.ndev, st);
    if (rc == TS_ERR_TOO_LARGE) {   // not cuttable: the whole span at once
      C10_CUDA_CHECK(cudaStreamSynchronize(st));
      c10::cuda::CUDACachingAllocator::raw_delete(staging);
      const int64_t span = ts_host_span_bytes(ctx->elem_bytes, shape.data(), strides.data(), (int)shape.size());
      staging = c10::cuda::CUDACachingAllocator::raw_alloc_with_stream(std::max<int64_t>(span, 16), st);
      rc = ts_copy_host_to_sticks(src.data_ptr(), staging, ctx->ptr, ctx->elem_bytes, shape.data(),
                                  strides.data(), (int)shape.size(), lay.dsize, lay.dstride, lay.dmap,
                                  lay.ndev, st);
    }
    // the host buffer must outlive the copy: wait for it unless the caller took that on
    if (!(non_blocking && rc == TS_OK && src_cpu.is_pinned())) C10_CUDA_CHECK(cudaStreamSynchronize(st));
    c10::cuda::CUDACachingAllocator::raw_delete(staging);
    check_status(rc, "copy host to device");
    return;
  }
  // destination is a view: patch the row-major form of its base and lay it out again
  at::Tensor raw = base_to_rowmajor(dst);
  view_in(raw, dst).copy_(src);
  rowmajor_to_base(raw, dst);
}

void device_to_host(const at::Tensor& src, const at::Tensor& dst_cpu) {
  StorageCtx* ctx = storage_ctx(src);
  const c10::cuda::CUDAGuard guard(ctx->device);
  if (src.numel() == 0) return;
  cudaStream_t st = current_stream(ctx->device);
  const bool same_shape = src.sizes() == dst_cpu.sizes() ||
                          (src.dim() == 1 && dst_cpu.dim() == 0 && src.numel() == 1);
  bool nonneg = true;
  for (auto s : dst_cpu.strides()) nonneg = nonneg && s > 0;
  if (is_canonical(src) && same_shape && (nonneg || dst_cpu.numel() == 1)) {
    auto shape = src.sizes().vec();
    if (shape.empty()) shape = {1};
    auto strides = dst_cpu.strides().vec();
    if (strides.size() != shape.size()) strides.assign(shape.size(), 1);
    const int64_t span = ts_host_span_bytes(ctx->elem_bytes, shape.data(), strides.data(), (int)shape.size());
    const auto lay = layout_of(shape, ctx->elem_bytes);
    int64_t dense = ctx->elem_bytes;
    for (auto s : shape) dense *= s;
    void* staging = nullptr;
    int rc = TS_ERR_TOO_LARGE;
    if (span == dense) {   // chunks through a small staging block, relayout and copy overlapped
      const int64_t want = std::max<int64_t>(
          ts_copy_staging_bytes(ctx->elem_bytes, shape.data(), strides.data(), (int)shape.size()), 256);
      staging = c10::cuda::CUDACachingAllocator::raw_alloc_with_stream(want, st);
      rc = ts_copy_sticks_to_host_pipelined(ctx->ptr, staging, want, dst_cpu.data_ptr(), ctx->elem_bytes,
                                            shape.data(), strides.data(), (int)shape.size(), lay.dsize,
                                            lay.dstride, lay.dmap, lay.ndev, st);
      if (rc == TS_ERR_TOO_LARGE) {
        C10_CUDA_CHECK(cudaStreamSynchronize(st));
        c10::cuda::CUDACachingAllocator::raw_delete(staging);
        staging = nullptr;
      }
    }
    if (rc == TS_ERR_TOO_LARGE) {
      staging = c10::cuda::CUDACachingAllocator::raw_alloc_with_stream(std::max<int64_t>(span, 16), st);
      // a destination with gaps keeps its gap bytes: pre-load the staging image with them
      if (span != dense)
        C10_CUDA_CHECK(cudaMemcpyAsync(staging, dst_cpu.data_ptr(), span, cudaMemcpyHostToDevice, st));
      rc = ts_copy_sticks_to_host(ctx->ptr, staging, dst_cpu.data_ptr(), ctx->elem_bytes, shape.data(),
                                  strides.data(), (int)shape.size(), lay.dsize, lay.dstride, lay.dmap,
                                  lay.ndev, st);
    }
    C10_CUDA_CHECK(cudaStreamSynchronize(st));
    c10::cuda::CUDACachingAllocator::raw_delete(staging);
    check_status(rc, "copy device to host");
    return;
  }
  at::Tensor raw = base_to_rowmajor(src);
  dst_cpu.copy_(view_in(raw, src));
}

// One pass, image to image, when both tensors are views the restickify kernel can walk.
bool restickify(const at::Tensor& src, const at::Tensor& dst) {
  StorageCtx* sctx = storage_ctx(src);
  StorageCtx* dctx = storage_ctx(dst);
  if (sctx->device != dctx->device || sctx->elem_bytes != dctx->elem_bytes) return false;
  if (sctx->ptr == dctx->ptr) return false;            // overlapping images: take the two-pass route
  auto size = dst.sizes().vec();
  at::Tensor s = src.sizes() == dst.sizes() ? src : src.expand(dst.sizes());
  auto sstr = s.strides().vec(), dstr = dst.strides().vec();
  if (size.empty()) { size = {1}; sstr = {1}; dstr = {1}; }
  if ((int)size.size() > TS_MAX_DIMS) return false;
  const int rc = ts_transpose_tiles(sctx->ptr, sctx->base_shape.data(), (int)sctx->base_shape.size(),
                                    sstr.data(), s.storage_offset(), dctx->ptr, dctx->base_shape.data(),
                                    (int)dctx->base_shape.size(), dstr.data(), dst.storage_offset(),
                                    size.data(), (int)size.size(), dctx->elem_bytes,
                                    current_stream(dctx->device));
  if (rc == TS_ERR_UNSUPPORTED) return false;
  check_status(rc, "restickify");
  return true;
}

void device_to_device(const at::Tensor& src, const at::Tensor& dst) {
  StorageCtx* sctx = storage_ctx(src);
  StorageCtx* dctx = storage_ctx(dst);
  const c10::cuda::CUDAGuard guard(dctx->device);
  if (dst.numel() == 0) return;
  if (is_canonical(src) && is_canonical(dst) && src.sizes() == dst.sizes()) {
    C10_CUDA_CHECK(cudaMemcpyAsync(dctx->ptr, sctx->ptr, stick_nbytes(dctx->base_shape, dctx->elem_bytes),
                                   cudaMemcpyDefault, current_stream(dctx->device)));
    return;
  }
  if (restickify_enabled()) {
    if (restickify(src, dst)) return;
    if (!is_canonical(dst) && !is_canonical(src)) {
      // the source is a view the one-pass kernel cannot walk: give it its own image first (two
      // passes over the source only), then write that image into the destination view
      at::Tensor tmp = at::empty(dst.sizes(), src.options());
      device_to_device(src, tmp);
      if (restickify(tmp, dst)) return;
    }
  }
  at::Tensor sraw = base_to_rowmajor(src);
  at::Tensor sview = view_in(sraw, src);
  if (is_canonical(dst)) {
    at::Tensor dense = sview.expand(dst.sizes()).to(at::Device(at::kCUDA, dctx->device));
    auto shape = dst.sizes().vec();
    auto strides = dense.strides().vec();
    if (shape.empty()) { shape = {1}; strides = {1}; }
    const auto lay = layout_of(shape, dctx->elem_bytes);
    check_status(ts_relayout_to_sticks(dense.data_ptr(), dctx->ptr, dctx->elem_bytes, shape.data(),
                                       strides.data(), (int)shape.size(), lay.dsize, lay.dstride,
                                       lay.dmap, lay.ndev, current_stream(dctx->device)),
                 "relayout to sticks");
    // `dense` is freed to the caching allocator in stream order
    return;
  }
  at::Tensor draw = base_to_rowmajor(dst);
  view_in(draw, dst).copy_(sview);
  rowmajor_to_base(draw, dst);
}

}  // namespace

// Test hook: route device-to-device copies of views through the two-pass path instead.
static bool g_restickify = true;
bool restickify_enabled() { return g_restickify; }
void set_restickify_enabled(bool on) { g_restickify = on; }

namespace {

at::Tensor spyre_copy_from(const at::Tensor& self, const at::Tensor& dst, bool non_blocking) {
  TORCH_CHECK(self.scalar_type() == dst.scalar_type(),
              "Spyre backend does not support type conversion yet during copy.");
  if (self.is_cpu() && dst.is_privateuseone()) {
    host_to_device(self, dst, non_blocking);
  } else if (self.is_privateuseone() && dst.is_cpu()) {
    device_to_host(self, dst);
  } else if (self.is_privateuseone() && dst.is_privateuseone()) {
    device_to_device(self, dst);
  } else {
    TORCH_CHECK(false, "spyre copy between ", self.device(), " and ", dst.device(),
                " is not supported");
  }
  return dst;
}

at::Tensor spyre_copy_from_and_resize(const at::Tensor& self, const at::Tensor& dst) {
  TORCH_CHECK(self.sizes() == dst.sizes() || dst.numel() == 0,
              "_copy_from_and_resize: size mismatch");
  if (dst.numel() == 0 && self.numel() != 0) {
    TORCH_CHECK(dst.is_cpu(), "cannot resize a spyre tensor");
    at::native::resize_output(dst, self.sizes());
  }
  return spyre_copy_from(self, dst, false);
}

at::Scalar spyre_local_scalar_dense(const at::Tensor& self) {
  TORCH_CHECK(self.numel() == 1, "a Tensor with ", self.numel(),
              " elements cannot be converted to Scalar");
  at::Tensor host = at::empty(self.sizes(), self.options().device(at::kCPU));
  device_to_host(self, host);
  return host.item();
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("empty.memory_format", TORCH_FN(spyre_empty));
  m.impl("empty_strided", TORCH_FN(spyre_empty_strided));
  m.impl("as_strided", TORCH_FN(spyre_as_strided));
  m.impl("set_.source_Storage_storage_offset", TORCH_FN(spyre_set_storage));
  m.impl("view", TORCH_FN(spyre_view));
  m.impl("_reshape_alias", TORCH_FN(spyre_reshape_alias));
  m.impl("_copy_from", TORCH_FN(spyre_copy_from));
  m.impl("_copy_from_and_resize", TORCH_FN(spyre_copy_from_and_resize));
  m.impl("_local_scalar_dense", TORCH_FN(spyre_local_scalar_dense));
}

}  // namespace spyre
