#include "eux/axon/axon_runtime.hpp"

namespace eux::axon {

AxonRuntime::AxonRuntime(std::string worker_name, size_t thread_pool_size, std::chrono::milliseconds timeout,
                         std::unique_ptr<ucxx::UcxAutoDeviceContext> device_context, std::shared_ptr<ucxx::UcxMemoryResourceManager> mr)
    : mr_(std::move(mr)) {
  if (!mr_) mr_ = std::make_shared<ucxx::DefaultUcxMemoryResourceManager>();
  // a worker always has a device context; without one from the caller it is the no-op one
  if (!device_context) device_context = std::make_unique<ucxx::UcxAutoDefaultDeviceContext>();
  worker_ = std::make_unique<AxonWorker>(mr_, std::move(worker_name), thread_pool_size, timeout, std::move(device_context));
}

AxonRuntime::~AxonRuntime() {
  if (worker_) worker_->Stop();
}

}  // namespace eux::axon
