// Header-only NVTX3 ranges (no link-time dependency; the reference links the
// legacy nvToolsExt library, reference: CMakeLists.txt:23).  One range named
// "mini_ncclAllReduce" (ARGB 0xFFFF0000) per AllReduce as in the reference
// (reference: src/api.cpp:143-151) stays in the default domain; new are the payload
// (element count) and a second range per launch in the domain "Mini-NCCL" whose name
// is the collective and the algorithm chosen and whose payload is the message size.
#pragma once
#include <cstdint>

#if __has_include(<nvtx3/nvToolsExt.h>) && !defined(MNCCL_NO_NVTX)
#include <nvtx3/nvToolsExt.h>
#define MNCCL_HAVE_NVTX 1
#else
#define MNCCL_HAVE_NVTX 0
#endif

namespace mnccl {

class NvtxRange {
 public:
  NvtxRange(const char* name, uint32_t argb, uint64_t payload = 0) {
#if MNCCL_HAVE_NVTX
    nvtxEventAttributes_t a = {};
    a.version = NVTX_VERSION;
    a.size = NVTX_EVENT_ATTRIB_STRUCT_SIZE;
    a.colorType = NVTX_COLOR_ARGB;
    a.color = argb;
    a.messageType = NVTX_MESSAGE_TYPE_ASCII;
    a.message.ascii = name;
    a.payloadType = NVTX_PAYLOAD_TYPE_UNSIGNED_INT64;
    a.payload.ullValue = payload;
    nvtxRangePushEx(&a);
#else
    (void)name; (void)argb; (void)payload;
#endif
  }
  ~NvtxRange() {
#if MNCCL_HAVE_NVTX
    nvtxRangePop();  // popped on every exit path, including exceptions
#endif
  }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

// A range in the library's own domain (created on first use): tools can filter on it.
class NvtxDomainRange {
 public:
  NvtxDomainRange(const char* name, uint64_t payload) {
#if MNCCL_HAVE_NVTX
    static nvtxDomainHandle_t domain = nvtxDomainCreateA("Mini-NCCL");
    domain_ = domain;
    nvtxEventAttributes_t a = {};
    a.version = NVTX_VERSION;
    a.size = NVTX_EVENT_ATTRIB_STRUCT_SIZE;
    a.messageType = NVTX_MESSAGE_TYPE_ASCII;
    a.message.ascii = name;
    a.payloadType = NVTX_PAYLOAD_TYPE_UNSIGNED_INT64;
    a.payload.ullValue = payload;
    nvtxDomainRangePushEx(domain_, &a);
#else
    (void)name; (void)payload;
#endif
  }
  ~NvtxDomainRange() {
#if MNCCL_HAVE_NVTX
    nvtxDomainRangePop(domain_);
#endif
  }
  NvtxDomainRange(const NvtxDomainRange&) = delete;
  NvtxDomainRange& operator=(const NvtxDomainRange&) = delete;

 private:
#if MNCCL_HAVE_NVTX
  nvtxDomainHandle_t domain_ = nullptr;
#endif
};

}  // namespace mnccl
