#include "core/error.h"
#include "core/log.h"
#include "net/soft_transport.h"
#include "net/transport.h"

#if defined(MNCCL_HAVE_VERBS)
#include "net/verbs_transport.h"
#endif

namespace mnccl {

bool verbs_compiled_in() {
#if defined(MNCCL_HAVE_VERBS)
  return true;
#else
  return false;
#endif
}

std::unique_ptr<OneSidedTransport> make_transport(const std::string& kind, int rank, int size) {
  if (kind == "verbs") {
#if defined(MNCCL_HAVE_VERBS)
    return std::unique_ptr<OneSidedTransport>(new VerbsTransport(rank, size));
#else
    fail(Result::SystemError, "MINI_NCCL_TRANSPORT=verbs, but this build has no libibverbs support "
                              "(<infiniband/verbs.h> was not found at build time)");
#endif
  }
  if (kind == "auto") {
#if defined(MNCCL_HAVE_VERBS)
    try {
      return std::unique_ptr<OneSidedTransport>(new VerbsTransport(rank, size));
    } catch (const std::exception& e) {
      MNCCL_INFO("Mini-NCCL", "verbs transport unavailable (%s); using the soft transport", e.what());
    }
#endif
    return std::unique_ptr<OneSidedTransport>(new SoftTransport(rank, size));
  }
  if (kind == "soft") return std::unique_ptr<OneSidedTransport>(new SoftTransport(rank, size));
  fail(Result::InvalidArgument, "unknown transport '" + kind + "'");
}

}  // namespace mnccl
