// Logging, CUDA error checks and raw .bin file I/O of the host-side operator layer
// (the role of utils/utils.h in the reference: INFO_LOG/ERROR_LOG, ACL_CHECK, ReadFile, WriteFile).
#ifndef CATCCOS_HOST_UTILS_H
#define CATCCOS_HOST_UTILS_H

#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/file.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>
#include <fstream>
#include <string>

#define INFO_LOG(fmt, ...) std::fprintf(stdout, "[INFO]  " fmt "\n", ##__VA_ARGS__)
#define WARN_LOG(fmt, ...) std::fprintf(stdout, "[WARN]  " fmt "\n", ##__VA_ARGS__)
#define ERROR_LOG(fmt, ...) std::fprintf(stderr, "[ERROR] " fmt "\n", ##__VA_ARGS__)

// Same contract as the reference's ACL_CHECK (utils/utils.h:26-32): report file:line and carry on.
#define CUDA_CHECK(call)                                                                          \
    do {                                                                                          \
        cudaError_t _e = (call);                                                                  \
        if (_e != cudaSuccess)                                                                    \
            std::fprintf(stderr, "%s:%d cudaError: %s\n", __FILE__, __LINE__, cudaGetErrorString(_e)); \
    } while (0)

inline bool ReadFile(const std::string &path, void *buffer, size_t bufferSize) {
    struct stat sb;
    if (stat(path.c_str(), &sb) == -1 || !S_ISREG(sb.st_mode)) {
        ERROR_LOG("%s is not a readable file", path.c_str());
        return false;
    }
    std::ifstream f(path, std::ios::binary);
    if (!f.is_open()) {
        ERROR_LOG("Open file failed. path = %s", path.c_str());
        return false;
    }
    const size_t size = static_cast<size_t>(sb.st_size);
    if (size == 0 || size > bufferSize) {
        ERROR_LOG("%s holds %zu bytes, the buffer %zu", path.c_str(), size, bufferSize);
        return false;
    }
    f.read(static_cast<char *>(buffer), static_cast<std::streamsize>(size));
    return static_cast<size_t>(f.gcount()) == size;
}

// Writes `size` bytes at byte `offset`, holding an exclusive lock so that several ranks can fill one file
// (Matmul-ReduceScatter writes rank r at offset r*size, as the reference does).
inline bool WriteFile(const std::string &path, const void *buffer, size_t size, size_t offset = 0) {
    if (buffer == nullptr) {
        ERROR_LOG("Write file failed. Buffer is nullptr.");
        return false;
    }
    const int fd = open(path.c_str(), O_RDWR | O_CREAT, 0666);
    if (fd == -1) {
        ERROR_LOG("Open file failed. path = %s", path.c_str());
        return false;
    }
    bool ok = flock(fd, LOCK_EX) == 0 && lseek(fd, static_cast<off_t>(offset), SEEK_SET) != -1;
    const char *p = static_cast<const char *>(buffer);
    size_t left = size;
    while (ok && left > 0) {
        const ssize_t n = write(fd, p, left);
        if (n <= 0) ok = false;
        else { p += n; left -= static_cast<size_t>(n); }
    }
    flock(fd, LOCK_UN);
    close(fd);
    if (!ok) ERROR_LOG("Write file failed. path = %s (%s)", path.c_str(), strerror(errno));
    return ok;
}

#endif  // CATCCOS_HOST_UTILS_H
