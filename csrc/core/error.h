// Error type used inside the library.  Every ABI entry point converts it (and
// any other exception) into an ncclResult_t: the "exception firewall" of the
// reference (reference: src/api.cpp:62-65,182-189), with a richer mapping.
#pragma once
#include <stdexcept>
#include <string>

namespace mnccl {

// Mirrors ncclResult_t numerically (kept separate so host-only code does not
// need the CUDA-including public header).
enum class Result : int {
  Success = 0,
  UnhandledCudaError = 1,
  SystemError = 2,
  InternalError = 3,
  InvalidArgument = 4,
  InvalidUsage = 5,
  RemoteError = 6,
  InProgress = 7
};

class Error : public std::runtime_error {
 public:
  Error(Result code, const std::string& what) : std::runtime_error(what), code_(code) {}
  Result code() const { return code_; }

 private:
  Result code_;
};

[[noreturn]] inline void fail(Result code, const std::string& what) { throw Error(code, what); }

#define MNCCL_CHECK_ARG(cond, msg)                                              \
  do {                                                                          \
    if (!(cond)) ::mnccl::fail(::mnccl::Result::InvalidArgument, (msg));        \
  } while (0)

}  // namespace mnccl
