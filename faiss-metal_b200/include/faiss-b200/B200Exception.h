// Exceptions of the B200 backend.  The reference throws faiss::FaissException for argument
// errors (src/MetalIndexFlat.mm:321-326,509-511; src/MetalSelect.mm:67-70) and
// std::runtime_error for device / allocation / library failures
// (src/StandardMetalResources.mm:21-23,71-74).  Both are kept as the base classes, so a caller
// written against the reference catches what it always caught; the subclasses add the status
// code of the C-ABI (B200F_ERR_* in b200_flat.h), which the handle-based C mirror returns
// without having to read the message.
#pragma once
#include <faiss/impl/FaissAssert.h>

#include <stdexcept>
#include <string>

namespace faiss_b200 {

/// Bad argument, unsupported size, key out of range, consumed token.
class B200ArgumentError : public faiss::FaissException {
   public:
    B200ArgumentError(int status, const std::string& msg) : faiss::FaissException(msg), status_(status) {}
    int status() const { return status_; }

   private:
    int status_;
};

/// CUDA failure, out of memory, no usable device, device-side status.
class B200RuntimeError : public std::runtime_error {
   public:
    B200RuntimeError(int status, const std::string& msg) : std::runtime_error(msg), status_(status) {}
    int status() const { return status_; }

   private:
    int status_;
};

}  // namespace faiss_b200

#define B200_THROW_ARG_IF_NOT(STATUS, COND, MSG)                                   \
    do {                                                                            \
        if (!(COND)) throw faiss_b200::B200ArgumentError((STATUS), std::string("faiss-b200: ") + (MSG)); \
    } while (false)
