// Minimal stand-in for <faiss/impl/FaissAssert.h> (see ../MetricType.h).
// Provides faiss::FaissException and the two throw macros the reference uses
// (src/MetalIndexFlat.mm:321-326,509-511; src/MetalSelect.mm:67-70).
#pragma once
#include <cstdio>
#include <exception>
#include <string>

namespace faiss {

class FaissException : public std::exception {
   public:
    explicit FaissException(const std::string& m) : msg(m) {}
    FaissException(const std::string& m, const char* func, const char* file, int line) {
        msg = std::string("Error in ") + func + " at " + file + ":" + std::to_string(line) + ": " + m;
    }
    const char* what() const noexcept override { return msg.c_str(); }
    std::string msg;
};

}  // namespace faiss

#define FAISS_THROW_MSG(MSG) \
    do { throw faiss::FaissException(MSG, __PRETTY_FUNCTION__, __FILE__, __LINE__); } while (false)

#define FAISS_THROW_FMT(FMT, ...)                                             \
    do {                                                                      \
        std::string __s;                                                      \
        int __size = std::snprintf(nullptr, 0, FMT, __VA_ARGS__);             \
        __s.resize(__size + 1);                                               \
        std::snprintf(&__s[0], __s.size(), FMT, __VA_ARGS__);                 \
        __s.resize(__size);                                                   \
        throw faiss::FaissException(__s, __PRETTY_FUNCTION__, __FILE__, __LINE__); \
    } while (false)

#define FAISS_THROW_IF_NOT_MSG(X, MSG) \
    do { if (!(X)) { FAISS_THROW_MSG(MSG); } } while (false)

#define FAISS_THROW_IF_NOT_FMT(X, FMT, ...) \
    do { if (!(X)) { FAISS_THROW_FMT(FMT, __VA_ARGS__); } } while (false)

#define FAISS_THROW_IF_NOT(X) FAISS_THROW_IF_NOT_MSG(X, "assertion '" #X "' failed")
