// Minimal stand-in for Faiss' exception type and assertion macros (NOT Faiss).
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
#define FAISS_THROW_MSG(MSG) throw ::faiss::FaissException(MSG, __func__, __FILE__, __LINE__)
#define FAISS_THROW_FMT(FMT, ...)                                   \
    do {                                                            \
        char _b[1024];                                              \
        std::snprintf(_b, sizeof(_b), FMT, __VA_ARGS__);            \
        throw ::faiss::FaissException(_b, __func__, __FILE__, __LINE__); \
    } while (0)
#define FAISS_THROW_IF_NOT_MSG(X, MSG) do { if (!(X)) FAISS_THROW_MSG(MSG); } while (0)
#define FAISS_THROW_IF_NOT_FMT(X, FMT, ...) do { if (!(X)) FAISS_THROW_FMT(FMT, __VA_ARGS__); } while (0)
#define FAISS_THROW_IF_NOT(X) FAISS_THROW_IF_NOT_MSG(X, "assertion '" #X "' failed")
