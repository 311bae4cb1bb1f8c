#pragma once
namespace llis { namespace ipc {
template <typename T> class ShmPrimitiveChannelGpu {};
class ShmChannelCpuReader {};
} }
