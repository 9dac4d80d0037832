// `spyre` (PrivateUse1) device core on CUDA memory: allocator, device guard, hooks.
//
// Mirrors the registrations of the reference's device core
// (torch_spyre/csrc/spyre_mem.cpp:440-554 allocator and guard,
// torch_spyre/csrc/spyre_hooks.cpp:33-259 hooks and stream/event methods), with the
// flex runtime replaced by CUDA: `spyre:N` is CUDA device N, streams and events are
// the CUDA ones PyTorch manages.
#include <ATen/Context.h>
#include <ATen/cuda/CUDAContext.h>
#include <ATen/detail/CUDAHooksInterface.h>
#include <ATen/detail/PrivateUse1HooksInterface.h>
#include <c10/core/impl/DeviceGuardImplInterface.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAFunctions.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <cstdlib>

#include "spyre_storage.h"

namespace spyre {

// ---- logging: TORCH_SPYRE_DEBUG, as torch_spyre/csrc/logging.h:56-61 ----------------
static bool g_debug = false;
void register_debug_flag() {
  const char* v = std::getenv("TORCH_SPYRE_DEBUG");
  g_debug = v && std::atoi(v) != 0;
}
bool debug_enabled() { return g_debug; }

int64_t stick_nbytes(c10::IntArrayRef shape, int64_t elem_bytes) {
  if (shape.empty()) return kBytesInStick;
  int64_t rows = 1;
  for (size_t i = 0; i + 1 < shape.size(); ++i) rows *= shape[i];
  const int64_t per_stick = kBytesInStick / elem_bytes;
  const int64_t sticks = (shape.back() + per_stick - 1) / per_stick;
  return sticks * rows * kBytesInStick;
}

// ---- allocator ---------------------------------------------------------------------
namespace {

void delete_ctx(void* ctx_void) {
  auto* ctx = static_cast<StorageCtx*>(ctx_void);
  if (!ctx) return;
  if (ctx->ptr) {
    c10::cuda::CUDAGuard guard(ctx->device);
    c10::cuda::CUDACachingAllocator::raw_delete(ctx->ptr);
  }
  delete ctx;
}

struct SpyreAllocator final : public at::Allocator {
  at::DataPtr allocate(size_t nbytes) override {
    // PyTorch brings CUDA (and its caching allocator) up lazily; make sure it has.
    at::globalContext().lazyInitDevice(c10::DeviceType::CUDA);
    const c10::DeviceIndex dev = c10::cuda::current_device();
    const c10::Device device(c10::DeviceType::PrivateUse1, dev);
    auto* ctx = new StorageCtx();
    ctx->device = dev;
    ctx->nbytes = nbytes;
    if (nbytes > 0) {
      // whole sticks, so that kernels may always touch full 128-byte lines
      const size_t padded = (nbytes + kBytesInStick - 1) / kBytesInStick * kBytesInStick;
      ctx->ptr = c10::cuda::CUDACachingAllocator::raw_alloc_with_stream(
          padded, c10::cuda::getCurrentCUDAStream(dev));
      TORCH_CHECK(ctx->ptr, "Failed to allocate ", nbytes, " bytes on Spyre device.");
    }
    return at::DataPtr(ctx->ptr, ctx, &delete_ctx, device);
  }
  // Only the context knows how to free an allocation (spyre_mem.cpp:540-542).
  at::DeleterFnPtr raw_deleter() const override { return nullptr; }
  void copy_data(void* dest, const void* src, std::size_t count) const final {
    C10_CUDA_CHECK(cudaMemcpyAsync(dest, src, count, cudaMemcpyDeviceToDevice,
                                   c10::cuda::getCurrentCUDAStream()));
  }
};

SpyreAllocator g_allocator;

}  // namespace

at::Allocator* spyre_allocator() { return &g_allocator; }
REGISTER_ALLOCATOR(c10::DeviceType::PrivateUse1, &g_allocator);

StorageCtx* storage_ctx(const at::Tensor& t) {
  TORCH_CHECK(t.device().is_privateuseone(), "expected a spyre tensor, got ", t.device());
  auto* ctx = static_cast<StorageCtx*>(t.storage().data_ptr().get_context());
  TORCH_CHECK(ctx, "spyre tensor without a device allocation");
  return ctx;
}

bool is_canonical(const at::Tensor& t) {
  if (!t.is_contiguous() || t.storage_offset() != 0) return false;
  const StorageCtx* ctx = storage_ctx(t);
  if (ctx->elem_bytes != (int)t.element_size()) return false;
  const auto& base = ctx->base_shape;
  int64_t base_numel = 1;
  for (auto s : base) base_numel *= s;
  if (base_numel != t.numel()) return false;
  if (t.numel() == 0) return true;
  const int64_t base_cols = base.empty() ? 1 : base.back();
  const int64_t cols = t.dim() ? t.size(-1) : 1;
  return base_cols == cols;
}

at::Tensor storage_as_cuda_bytes(const at::Tensor& t) {
  StorageCtx* ctx = storage_ctx(t);
  const int64_t n = stick_nbytes(ctx->base_shape, ctx->elem_bytes ? ctx->elem_bytes : 1);
  c10::Storage keep = t.storage();
  auto opts = at::TensorOptions().dtype(at::kByte).device(at::Device(at::kCUDA, ctx->device));
  return at::from_blob(ctx->ptr, {ctx->ptr ? n : 0}, [keep](void*) mutable { keep = c10::Storage(); },
                       opts);
}

// ---- device guard: spyre:N <-> cuda:N ------------------------------------------------
namespace {

struct SpyreGuardImpl final : c10::impl::DeviceGuardImplInterface {
  static c10::Device dev(c10::DeviceIndex i) { return {c10::DeviceType::PrivateUse1, i}; }
  static c10::Stream wrap(const c10::cuda::CUDAStream& s) {
    return c10::Stream(c10::Stream::UNSAFE, dev(s.device_index()), s.id());
  }
  static c10::cuda::CUDAStream unwrap(const c10::Stream& s) {
    return c10::cuda::CUDAStream(c10::Stream(
        c10::Stream::UNSAFE, c10::Device(c10::DeviceType::CUDA, s.device_index()), s.id()));
  }
  c10::DeviceType type() const override { return c10::DeviceType::PrivateUse1; }
  c10::Device exchangeDevice(c10::Device d) const override {
    const auto old = getDevice();
    setDevice(d);
    return old;
  }
  c10::Device getDevice() const override { return dev(c10::cuda::current_device()); }
  void setDevice(c10::Device d) const override {
    TORCH_INTERNAL_ASSERT(d.is_privateuseone());
    if (d.index() >= 0) c10::cuda::set_device(d.index());
  }
  void uncheckedSetDevice(c10::Device d) const noexcept override {
    if (d.index() >= 0) c10::cuda::MaybeSetDevice(d.index());
  }
  c10::DeviceIndex deviceCount() const noexcept override { return c10::cuda::device_count(); }
  c10::Stream getStream(c10::Device d) const override {
    return wrap(c10::cuda::getCurrentCUDAStream(d.index()));
  }
  c10::Stream getDefaultStream(c10::Device d) const override {
    return wrap(c10::cuda::getDefaultCUDAStream(d.index()));
  }
  c10::Stream getNewStream(c10::Device d, int priority = 0) const override {
    return wrap(c10::cuda::getStreamFromPool(priority, d.index()));
  }
  c10::Stream exchangeStream(c10::Stream s) const override {
    const auto cs = unwrap(s);
    const auto old = c10::cuda::getCurrentCUDAStream(cs.device_index());
    c10::cuda::setCurrentCUDAStream(cs);
    return wrap(old);
  }
  bool queryStream(const c10::Stream& s) const override { return unwrap(s).query(); }
  void synchronizeStream(const c10::Stream& s) const override { unwrap(s).synchronize(); }
  void synchronizeDevice(const c10::DeviceIndex i) const override {
    c10::cuda::CUDAGuard guard(i);
    c10::cuda::device_synchronize();
  }
  void recordDataPtrOnStream(const c10::DataPtr&, const c10::Stream&) const override {}
  void* getStreamNativeHandle(const c10::Stream s) const override { return unwrap(s).stream(); }

  // ---- events: CUDA events behind c10::Event, as the reference's guard implements them on its
  // own runtime (torch_spyre/csrc/spyre_hooks.cpp:108-256: record, block, queryEvent,
  // elapsedTime, destroyEvent).  An event is created lazily by its first record().
  void destroyEvent(void* event, const c10::DeviceIndex device_index) const noexcept override {
    if (!event) return;
    int orig = -1;
    if (cudaGetDevice(&orig) != cudaSuccess) return;
    if (device_index >= 0) cudaSetDevice(device_index);
    cudaEventDestroy(static_cast<cudaEvent_t>(event));
    cudaSetDevice(orig);
  }
  void record(void** event, const c10::Stream& stream, const c10::DeviceIndex device_index,
              const c10::EventFlag flag) const override {
    TORCH_CHECK(device_index == -1 || device_index == stream.device_index(), "Event device index ",
                device_index, " does not match recording stream's device index ", stream.device_index(), ".");
    const c10::cuda::CUDAGuard guard(stream.device_index());
    auto ev = static_cast<cudaEvent_t>(*event);
    if (!ev) {
      unsigned int cuda_flag = cudaEventDisableTiming;
      switch (flag) {
        case c10::EventFlag::PYTORCH_DEFAULT: cuda_flag = cudaEventDisableTiming; break;
        case c10::EventFlag::BACKEND_DEFAULT: cuda_flag = cudaEventDefault; break;
        default: TORCH_CHECK(false, "spyre event received unknown flag");
      }
      C10_CUDA_CHECK(cudaEventCreateWithFlags(&ev, cuda_flag));
    }
    C10_CUDA_CHECK(cudaEventRecord(ev, unwrap(stream).stream()));
    *event = ev;
  }
  void block(void* event, const c10::Stream& stream) const override {
    if (!event) return;
    const c10::cuda::CUDAGuard guard(stream.device_index());
    C10_CUDA_CHECK(cudaStreamWaitEvent(unwrap(stream).stream(), static_cast<cudaEvent_t>(event), 0));
  }
  bool queryEvent(void* event) const override {
    if (!event) return true;
    const cudaError_t err = cudaEventQuery(static_cast<cudaEvent_t>(event));
    if (err == cudaErrorNotReady) {
      (void)cudaGetLastError();   // not ready is an answer, not an error
      return false;
    }
    C10_CUDA_CHECK(err);
    return true;
  }
  void synchronizeEvent(void* event) const override {
    if (!event) return;
    C10_CUDA_CHECK(cudaEventSynchronize(static_cast<cudaEvent_t>(event)));
  }
  double elapsedTime(void* event1, void* event2, const c10::DeviceIndex device_index) const override {
    TORCH_CHECK(event1 && event2, "Both events must be recorded before calculating elapsed time.");
    const c10::cuda::CUDAGuard guard(device_index >= 0 ? device_index : c10::cuda::current_device());
    float ms = 0;
    C10_CUDA_CHECK(cudaEventElapsedTime(&ms, static_cast<cudaEvent_t>(event1), static_cast<cudaEvent_t>(event2)));
    return static_cast<double>(ms);
  }
};

struct SpyreHooks final : at::PrivateUse1HooksInterface {
  bool isBuilt() const override { return true; }
  bool isAvailable() const override { return c10::cuda::device_count() > 0; }
  bool hasPrimaryContext(c10::DeviceIndex) const override { return true; }
  // pinned host memory is CUDA's
  at::Allocator* getPinnedMemoryAllocator() const override {
    return at::detail::getCUDAHooks().getPinnedMemoryAllocator();
  }
  bool isPinnedPtr(const void* data) const override {
    return at::detail::getCUDAHooks().isPinnedPtr(data);
  }
  at::Device getDeviceFromPtr(void* data) const override {
    cudaPointerAttributes attr{};
    C10_CUDA_CHECK(cudaPointerGetAttributes(&attr, data));
    return {c10::DeviceType::PrivateUse1, (c10::DeviceIndex)attr.device};
  }
  void resizePrivateUse1Bytes(const c10::Storage&, size_t) const override {
    TORCH_CHECK(false, "resizing a spyre storage is not supported");
  }
};

}  // namespace

C10_REGISTER_GUARD_IMPL(PrivateUse1, SpyreGuardImpl);

void register_hooks() {
  static SpyreHooks* hooks = new SpyreHooks();
  if (!at::isPrivateUse1HooksRegistered()) at::RegisterPrivateUse1HooksInterface(hooks);
}

}  // namespace spyre
