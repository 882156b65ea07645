#include "B200DeviceManager.h"
#include "B200Function.h"

#include "glow/Runtime/StatsExporter.h"

#include <cuda_runtime.h>

using namespace glow;
using namespace glow::runtime;

static Error toError(int rc) {
  if (rc == GLOWB200_OK) return Error::success();
  auto code = rc == GLOWB200_RUNTIME_NET_NOT_FOUND           ? ErrorValue::ErrorCode::RUNTIME_NET_NOT_FOUND
              : rc == GLOWB200_RUNTIME_OUT_OF_DEVICE_MEMORY  ? ErrorValue::ErrorCode::RUNTIME_OUT_OF_DEVICE_MEMORY
              : rc == GLOWB200_RUNTIME_DEVICE_NONRECOVERABLE ? ErrorValue::ErrorCode::RUNTIME_DEVICE_NONRECOVERABLE
                                                             : ErrorValue::ErrorCode::RUNTIME_ERROR;
  return MAKE_ERR(code, glowb200_last_error());
}

B200DeviceManager::B200DeviceManager(const DeviceConfig &config) : QueueBackedDeviceManager(config) {
  int ordinal = (int)config.deviceID;
  auto it = config.parameters.find("DeviceID");  // the key Glow's benchmarks use (tests/benchmark/CommonSLSEB.h:408-411)
  if (it != config.parameters.end()) ordinal = std::stoi(it->second);
  dm_ = glowb200_device_manager_create(ordinal, config.getDeviceMemory(0));
  glowb200_device_manager_set_context_count(dm_, 2);  // B200Backend::getContextCount
  statsExporterRegistry_->incrementCounter(kDevicesUsedB200);
}

B200DeviceManager::~B200DeviceManager() {
  ERR_TO_VOID(stop(true));
  glowb200_device_manager_destroy(dm_);
  statsExporterRegistry_->incrementCounter(kDevicesUsedB200, -1);
  zeroMemoryCounters();
}

Error B200DeviceManager::init() {
  // The CUDA context is created on the worker thread, not lazily in the first request.
  RETURN_IF_ERR(QueueBackedDeviceManager::init());
  std::promise<int> rc;
  workThread_.submit([&] { rc.set_value(glowb200_device_manager_init(dm_)); });
  RETURN_IF_ERR(toError(rc.get_future().get()));
  maxMemoryBytes_ = glowb200_device_manager_maximum_memory(dm_);
  exportMemoryCounters();
  return Error::success();
}

Error B200DeviceManager::stop(bool block) {
  glowb200_device_manager_stop(dm_);
  return QueueBackedDeviceManager::stop(block);
}

uint64_t B200DeviceManager::getMaximumMemory() const { return glowb200_device_manager_maximum_memory(dm_); }
uint64_t B200DeviceManager::getAvailableMemory() const { return glowb200_device_manager_available_memory(dm_); }
bool B200DeviceManager::isMemoryAvailable(uint64_t estimate) const { return glowb200_device_manager_is_memory_available(dm_, estimate); }

DeviceInfo B200DeviceManager::getDeviceInfo() const {
  // Peaks for the partitioner's cost model: measured copy bandwidth and library int8 GEMM rate.
  DeviceInfo info = DeviceInfo();
  info.availableMemory = getAvailableMemory();
  info.sramCapacity = 126ull * 1024 * 1024;     // L2
  info.peakCompute = 2.2e15;                    // int8 op/s the rowwise-FC kernel sustains (M2048 K4096 N4096, measured)
  info.peakDramBw = 6.5e12;                     // measured copy bandwidth
  info.peakSramBw = 2.0e13;
  info.peakPCIeBw = 4.2e10;                     // measured pinned host-to-device rate of a request
  return info;
}

void *B200DeviceManager::allocateDeviceIOBuffer(dim_t size) {
  void *p = nullptr;
  if (cudaHostAlloc(&p, size, cudaHostAllocDefault) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lock(bufferLock_);
  allocations_.insert(p);
  return p;
}

void B200DeviceManager::freeAllocatedDeviceIOBuffer(void *buffer) {
  std::lock_guard<std::mutex> lock(bufferLock_);
  if (allocations_.erase(buffer)) cudaFreeHost(buffer);
}

void B200DeviceManager::transferStaticPlaceholderToDevice(Placeholder *PH, Tensor *T, std::function<void(Error)> resultCB) {
  // every loaded function that names the placeholder gets the bytes (DeviceManager.h:163-171)
  workThread_.submit([this, PH, T, resultCB] {
    Error err = Error::success();
    for (const auto &func : functions_) {
      int rc = glowb200_device_manager_transfer_static_placeholder(dm_, func.first.c_str(), PH->getName().str().c_str(),
                                                                   T->getUnsafePtr(), T->getSizeInBytes());
      if (rc == GLOWB200_RUNTIME_ERROR) continue;  // this function does not use the placeholder
      if (rc != GLOWB200_OK) { err = toError(rc); break; }
    }
    resultCB(std::move(err));
  });
}

void *B200DeviceManager::placeholderAddress(const std::string &network, const std::string &placeholder) {
  void *p = nullptr;
  size_t bytes = 0;
  if (glowb200_device_manager_placeholder_address(dm_, network.c_str(), placeholder.c_str(), &p, &bytes) != GLOWB200_OK) return nullptr;
  return p;
}

// Device-resident tensors (DeviceManager.h:208-231).  \p locationContext is a device address
// inside a loaded network's placeholders (placeholderAddress).
void B200DeviceManager::transferToDevice(Tensor &tensor, void *locationContext, std::function<void(Error)> resultCB) {
  if (!locationContext) {
    resultCB(MAKE_ERR(ErrorValue::ErrorCode::RUNTIME_ERROR, "B200: transferToDevice needs the address of a placeholder"));
    return;
  }
  if (cudaMemcpy(locationContext, tensor.getUnsafePtr(), tensor.getUnpaddedSizeInBytes(), cudaMemcpyHostToDevice) != cudaSuccess) {
    resultCB(MAKE_ERR(ErrorValue::ErrorCode::RUNTIME_ERROR, std::string("B200: host-to-device copy failed: ") + cudaGetErrorString(cudaGetLastError())));
    return;
  }
  tensor.moveToDevice(this, locationContext);
  resultCB(Error::success());
}

void B200DeviceManager::transferFromDevice(Tensor &tensor, bool release, std::function<void(Error)> resultCB) {
  if (!tensor.isDeviceResident() || tensor.getDeviceManager() != this) {
    resultCB(MAKE_ERR(ErrorValue::ErrorCode::RUNTIME_ERROR, "B200: the tensor is not resident on this device"));
    return;
  }
  if (cudaMemcpy(tensor.getUnsafePtr(), tensor.getLocationContext(), tensor.getUnpaddedSizeInBytes(), cudaMemcpyDeviceToHost) != cudaSuccess) {
    resultCB(MAKE_ERR(ErrorValue::ErrorCode::RUNTIME_ERROR, std::string("B200: device-to-host copy failed: ") + cudaGetErrorString(cudaGetLastError())));
    return;
  }
  if (release) tensor.resetDeviceInfo();  // the memory itself belongs to the network's placeholder slab
  resultCB(Error::success());
}

bool B200DeviceManager::releaseDeviceTensor(void *) { return true; }  // nothing of its own to free

void B200DeviceManager::addNetworkImpl(const Module *module, FunctionMapTy functions, ReadyCBTy readyCB) {
  for (const auto &func : functions) {
    if (func.second->getCompileBackendName() != "B200") {
      readyCB(module, MAKE_ERR("Failed to add network: function " + func.first + " is not a B200Function"));
      return;
    }
  }
  for (const auto &func : functions) {
    auto *F = static_cast<B200Function *>(func.second);
    // translate + capture constants before the module may be stripped; an instruction without a
    // translation fails the network here, through the callback, and the host carries on
    if (auto err = F->translate(module)) {
      readyCB(module, std::move(err));
      return;
    }
    F->setDeviceManager(dm_, this);
    if (auto err = toError(glowb200_device_manager_add_network(dm_, F->handle()))) {
      readyCB(module, std::move(err));
      return;
    }
    functions_.emplace(func.first, func.second);
  }
  usedMemoryBytes_ = getMaximumMemory() - getAvailableMemory();
  exportMemoryCounters();
  readyCB(module, Error::success());
}

void B200DeviceManager::evictNetworkImpl(std::string functionName, EvictFunctionCBTy evictCB) {
  auto err = toError(glowb200_device_manager_evict_network(dm_, functionName.c_str()));
  if (!err) functions_.erase(functionName);
  usedMemoryBytes_ = getMaximumMemory() - getAvailableMemory();
  exportMemoryCounters();
  evictCB(functionName, std::move(err));
}

void B200DeviceManager::runFunctionImpl(RunIdentifierTy id, std::string function, std::unique_ptr<ExecutionContext> context,
                                        ResultCBTy resultCB) {
  TRACE_EVENT_SCOPE_NAMED(context->getTraceContext(), TraceLevel::RUNTIME, "DeviceManager::run", dmRun);
  auto it = functions_.find(function);
  if (it == functions_.end()) {
    TRACE_EVENT_SCOPE_END_NAMED(dmRun);
    resultCB(id, MAKE_ERR(ErrorValue::ErrorCode::RUNTIME_NET_NOT_FOUND, "Function " + function + " not found"), std::move(context));
    return;
  }
  auto err = it->second->execute(context.get());
  TRACE_EVENT_SCOPE_END_NAMED(dmRun);  // before the callback, as the CPU device manager does
  resultCB(id, std::move(err), std::move(context));
}
