#ifndef GLOW_BACKENDS_B200_B200DEVICEMANAGER_H
#define GLOW_BACKENDS_B200_B200DEVICEMANAGER_H

#include "glow/Backends/QueueBackedDeviceManager.h"

#include "glow_b200.h"

namespace glow {
namespace runtime {

/// One B200.  A single worker thread (QueueBackedDeviceManager) owns the CUDA device selection,
/// so everything enqueued for the device is stream-ordered.
class B200DeviceManager final : public QueueBackedDeviceManager {
  glowb200_device_manager *dm_{nullptr};
  FunctionMapTy functions_;
  static constexpr const char *kDevicesUsedB200 = "glow.devices_used.b200";

public:
  explicit B200DeviceManager(const DeviceConfig &config);
  ~B200DeviceManager() override;

  Error init() override;
  Error stop(bool block = true) override;
  uint64_t getMaximumMemory() const override;
  uint64_t getAvailableMemory() const override;
  bool isMemoryAvailable(uint64_t estimate) const override;
  DeviceInfo getDeviceInfo() const override;
  /// Pinned host memory for request I/O.
  void *allocateDeviceIOBuffer(dim_t size) override;
  void freeAllocatedDeviceIOBuffer(void *buffer) override;
  /// Static placeholders (embedding tables) are copied to the device once.
  void transferStaticPlaceholderToDevice(Placeholder *PH, Tensor *T, std::function<void(Error)> resultCB) override;

  /// Device-resident tensors: a tensor lives at the device address of a placeholder.
  void transferToDevice(Tensor &tensor, void *locationContext, std::function<void(Error)> resultCB = GLOW_DRT_DEFAULT_CB) override;
  void transferFromDevice(Tensor &tensor, bool release = true, std::function<void(Error)> resultCB = GLOW_DRT_DEFAULT_CB) override;
  bool releaseDeviceTensor(void *locationContext) override;
  /// Device address of a placeholder of a loaded network (context 0), or nullptr.
  void *placeholderAddress(const std::string &network, const std::string &placeholder);

protected:
  void addNetworkImpl(const Module *module, FunctionMapTy functions, ReadyCBTy cb) override;
  void evictNetworkImpl(std::string functionName, EvictFunctionCBTy evictCb) override;
  void runFunctionImpl(RunIdentifierTy id, std::string functionName, std::unique_ptr<ExecutionContext> context,
                       ResultCBTy cb) override;
};

} // namespace runtime
} // namespace glow
#endif
