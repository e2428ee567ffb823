// q8_file.cpp -- Q8_0 weights on disk, Q8_0R in device memory.
//
// The reference refuses to save quantized tensors (src/model/GGUF.cpp:204-213: save_gguf throws for them) and so
// re-quantizes every selected weight on the host at each start (PPMLModel::quantize_big_weight_matrices,
// src/model/PPML.cpp:4504-4524: device -> host fp32, quantize_q8_0_host, repack_q8_0_host, host -> device).  This
// file adds the missing piece: a writer that stores selected tensors as ggml Q8_0 blocks (type id 8, 34 bytes per 32
// elements: half scale + 32 int8, the layout of block_q8_0, include/ppml/QuantBlocks.h:33-36) next to fp32 tensors,
// and a loader that puts a Q8_0 tensor into device memory in the planar Q8_0R form the product kernels read
// ([numel] int8 plane, then [numel / 32] half scales), repacked on the device.
//
// The container is the reference's own GGUF dialect, so its reader walks the file unchanged up to the tensor type
// field: magic 0x46554747, version 3, 64-bit counts and string lengths, float32 / string metadata, a "layout_hash"
// string (FNV-1a over names and shapes, src/model/GGUF.cpp:28-72), tensor infos (name, n_dims, dims with the innermost
// first, type, offset), data aligned to 32 bytes.  As in the reference, tensor offsets are absolute file offsets.
// Quantization is the host rule of the reference (d = amax / 127 stored as half, q = round(x * (1 / d))), bit for bit.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/ppml_b200.h"

namespace {

constexpr uint32_t kMagic = 0x46554747u, kVersion = 3u;
constexpr size_t kAlign = 32;
constexpr uint32_t kTypeF32 = 0, kTypeQ8_0 = 8;           // ggml type ids
constexpr uint32_t kValF32 = 6, kValString = 8;           // metadata value types

size_t align_up(size_t n, size_t a) { return (n + a - 1) / a * a; }

struct Info {
    std::string name;
    std::vector<uint64_t> dims;       // innermost first, as the reference writes them
    uint32_t type = 0;
    uint64_t offset = 0;
    uint64_t numel() const { uint64_t n = 1; for (uint64_t d : dims) n *= d; return n; }
    uint64_t file_bytes() const { return type == kTypeQ8_0 ? numel() / 32 * 34 : numel() * 4; }
};

struct File {
    std::FILE* f = nullptr;
    std::vector<Info> tensors;
    std::string layout_hash;
};

uint64_t layout_hash(const std::vector<Info>& ts) {
    uint64_t h = 1469598103934665603ULL;
    auto feed = [&](uint8_t b) { h ^= b; h *= 1099511628211ULL; };
    auto feed32 = [&](uint32_t v) { for (int b = 0; b < 4; ++b) feed(static_cast<uint8_t>(v >> (8 * b))); };
    auto feed64 = [&](uint64_t v) { for (int b = 0; b < 8; ++b) feed(static_cast<uint8_t>(v >> (8 * b))); };
    for (const Info& t : ts) {
        for (char c : t.name) feed(static_cast<uint8_t>(c));
        feed32(0xFF);
        feed32(static_cast<uint32_t>(t.dims.size()));
        for (uint64_t d : t.dims) feed64(d);
        feed32(0xFE);
    }
    return h;
}

bool wr(std::FILE* f, const void* p, size_t n) { return n == 0 || std::fwrite(p, 1, n, f) == n; }
bool wr32(std::FILE* f, uint32_t v) { return wr(f, &v, 4); }
bool wr64(std::FILE* f, uint64_t v) { return wr(f, &v, 8); }
bool wrstr(std::FILE* f, const std::string& s) { return wr64(f, s.size()) && wr(f, s.data(), s.size()); }
bool pad_to(std::FILE* f, size_t pos, size_t target) {
    static const char zeros[64] = {0};
    while (pos < target) {
        const size_t n = target - pos < sizeof(zeros) ? target - pos : sizeof(zeros);
        if (!wr(f, zeros, n)) return false;
        pos += n;
    }
    return true;
}
bool rd(std::FILE* f, void* p, size_t n) { return n == 0 || std::fread(p, 1, n, f) == n; }
bool rdstr(std::FILE* f, std::string& s) {
    uint64_t n = 0;
    if (!rd(f, &n, 8) || n > (1u << 20)) return false;
    s.resize(static_cast<size_t>(n));
    return rd(f, &s[0], s.size());
}

}  // namespace

extern "C" {

int ppml_b200_q8_file_write(const char* path, int n_tensors, const char* const* names, const float* const* weights,
                            const int64_t* rows, const int64_t* cols, const int* as_q8) {
    if (!path || n_tensors <= 0 || !names || !weights || !rows || !cols || !as_q8) return 1;
    std::vector<Info> ts(static_cast<size_t>(n_tensors));
    for (int i = 0; i < n_tensors; ++i) {
        if (!names[i] || !weights[i] || rows[i] <= 0 || cols[i] <= 0) return 1;
        if (as_q8[i] && (cols[i] % 32) != 0) return 2;                 // blocks must not straddle rows
        ts[i].name = names[i];
        ts[i].dims = {static_cast<uint64_t>(cols[i]), static_cast<uint64_t>(rows[i])};
        ts[i].type = as_q8[i] ? kTypeQ8_0 : kTypeF32;
    }
    char hex[17];
    std::snprintf(hex, sizeof(hex), "%016llx", static_cast<unsigned long long>(layout_hash(ts)));
    const std::string hash_key = "layout_hash", hash_val = hex, fmt_key = "ppml_b200.q8_block", fmt_val = "ggml Q8_0 (half d + 32 x int8)";
    size_t head = 4 + 4 + 8 + 8;
    head += 8 + hash_key.size() + 4 + 8 + hash_val.size();
    head += 8 + fmt_key.size() + 4 + 8 + fmt_val.size();
    for (const Info& t : ts) head += 8 + t.name.size() + 4 + 8 * t.dims.size() + 4 + 8;
    size_t cur = align_up(head, kAlign);
    const size_t data_start = cur;
    for (Info& t : ts) { t.offset = cur; cur = align_up(cur + static_cast<size_t>(t.file_bytes()), kAlign); }

    std::FILE* f = std::fopen(path, "wb");
    if (!f) return 3;
    bool ok = wr32(f, kMagic) && wr32(f, kVersion) && wr64(f, static_cast<uint64_t>(n_tensors)) && wr64(f, 2);
    ok = ok && wrstr(f, hash_key) && wr32(f, kValString) && wrstr(f, hash_val);
    ok = ok && wrstr(f, fmt_key) && wr32(f, kValString) && wrstr(f, fmt_val);
    for (const Info& t : ts) {
        ok = ok && wrstr(f, t.name) && wr32(f, static_cast<uint32_t>(t.dims.size()));
        for (uint64_t d : t.dims) ok = ok && wr64(f, d);
        ok = ok && wr32(f, t.type) && wr64(f, t.offset);
    }
    ok = ok && pad_to(f, head, data_start);
    std::vector<uint8_t> blocks;
    for (int i = 0; ok && i < n_tensors; ++i) {
        const Info& t = ts[static_cast<size_t>(i)];
        const size_t bytes = static_cast<size_t>(t.file_bytes());
        if (t.type == kTypeQ8_0) {
            blocks.resize(bytes);
            if (ppml_b200_quantize_q8_0_host(weights[i], blocks.data(), static_cast<int64_t>(t.numel())) != 0) { ok = false; break; }
            ok = wr(f, blocks.data(), bytes);
        } else {
            ok = wr(f, weights[i], bytes);
        }
        ok = ok && pad_to(f, static_cast<size_t>(t.offset) + bytes, align_up(static_cast<size_t>(t.offset) + bytes, kAlign));
    }
    ok = (std::fclose(f) == 0) && ok;
    return ok ? 0 : 4;
}

void* ppml_b200_q8_file_open(const char* path) {
    if (!path) return nullptr;
    std::FILE* f = std::fopen(path, "rb");
    if (!f) return nullptr;
    File* h = new File();
    h->f = f;
    uint32_t magic = 0, version = 0;
    uint64_t n_tensors = 0, n_kv = 0;
    bool ok = rd(f, &magic, 4) && rd(f, &version, 4) && rd(f, &n_tensors, 8) && rd(f, &n_kv, 8) && magic == kMagic &&
              version == kVersion && n_tensors < (1u << 20) && n_kv < (1u << 20);
    for (uint64_t i = 0; ok && i < n_kv; ++i) {
        std::string key, val;
        uint32_t vt = 0;
        ok = rdstr(f, key) && rd(f, &vt, 4);
        if (!ok) break;
        if (vt == kValString) { ok = rdstr(f, val); if (key == "layout_hash") h->layout_hash = val; }
        else if (vt == 0 || vt == 1 || vt == 7) ok = std::fseek(f, 1, SEEK_CUR) == 0;
        else if (vt == 2 || vt == 3) ok = std::fseek(f, 2, SEEK_CUR) == 0;
        else if (vt == 4 || vt == 5 || vt == kValF32) ok = std::fseek(f, 4, SEEK_CUR) == 0;
        else if (vt == 10 || vt == 11 || vt == 12) ok = std::fseek(f, 8, SEEK_CUR) == 0;
        else ok = false;                                              // arrays are not written by either writer
    }
    h->tensors.resize(ok ? static_cast<size_t>(n_tensors) : 0);
    for (size_t i = 0; ok && i < h->tensors.size(); ++i) {
        Info& t = h->tensors[i];
        uint32_t nd = 0;
        ok = rdstr(f, t.name) && rd(f, &nd, 4) && nd >= 1 && nd <= 4;
        t.dims.resize(ok ? nd : 0);
        for (uint32_t d = 0; ok && d < nd; ++d) ok = rd(f, &t.dims[d], 8);
        ok = ok && rd(f, &t.type, 4) && rd(f, &t.offset, 8) && (t.type == kTypeF32 || t.type == kTypeQ8_0);
        if (ok && t.type == kTypeQ8_0 && (t.dims[0] % 32) != 0) ok = false;
    }
    if (!ok) { std::fclose(f); delete h; return nullptr; }
    return h;
}

void ppml_b200_q8_file_close(void* handle) {
    File* h = static_cast<File*>(handle);
    if (!h) return;
    if (h->f) std::fclose(h->f);
    delete h;
}

int ppml_b200_q8_file_count(void* handle) { return handle ? static_cast<int>(static_cast<File*>(handle)->tensors.size()) : -1; }

int ppml_b200_q8_file_find(void* handle, const char* name) {
    File* h = static_cast<File*>(handle);
    if (!h || !name) return -1;
    for (size_t i = 0; i < h->tensors.size(); ++i) if (h->tensors[i].name == name) return static_cast<int>(i);
    return -1;
}

int ppml_b200_q8_file_info(void* handle, int index, char* name, int name_cap, int64_t* rows, int64_t* cols, int* is_q8) {
    File* h = static_cast<File*>(handle);
    if (!h || index < 0 || static_cast<size_t>(index) >= h->tensors.size()) return 1;
    const Info& t = h->tensors[static_cast<size_t>(index)];
    if (name && name_cap > 0) { std::strncpy(name, t.name.c_str(), static_cast<size_t>(name_cap) - 1); name[name_cap - 1] = 0; }
    if (cols) *cols = static_cast<int64_t>(t.dims[0]);
    if (rows) *rows = static_cast<int64_t>(t.numel() / t.dims[0]);
    if (is_q8) *is_q8 = t.type == kTypeQ8_0 ? 1 : 0;
    return 0;
}

int64_t ppml_b200_q8_file_nbytes(void* handle, int index) {
    File* h = static_cast<File*>(handle);
    if (!h || index < 0 || static_cast<size_t>(index) >= h->tensors.size()) return -1;
    return static_cast<int64_t>(h->tensors[static_cast<size_t>(index)].file_bytes());      // Q8_0R takes the bytes of Q8_0
}

int ppml_b200_q8_file_layout_hash(void* handle, char* hex17) {
    File* h = static_cast<File*>(handle);
    if (!h || !hex17) return 1;
    std::strncpy(hex17, h->layout_hash.c_str(), 16);
    hex17[16] = 0;
    char want[17];
    std::snprintf(want, sizeof(want), "%016llx", static_cast<unsigned long long>(layout_hash(h->tensors)));
    return h->layout_hash == want ? 0 : 2;                            // 2: names / shapes do not match the stored hash
}

int ppml_b200_q8_file_load(void* handle, int index, void* dst_dev, void* scratch_dev, void* stream) {
    File* h = static_cast<File*>(handle);
    if (!h || !dst_dev || index < 0 || static_cast<size_t>(index) >= h->tensors.size()) return 1;
    const Info& t = h->tensors[static_cast<size_t>(index)];
    const size_t bytes = static_cast<size_t>(t.file_bytes());
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    void* host = nullptr;
    if (cudaMallocHost(&host, bytes) != cudaSuccess) { cudaGetLastError(); return 3; }
    int rc = 0;
    if (std::fseek(h->f, static_cast<long>(t.offset), SEEK_SET) != 0 || !rd(h->f, host, bytes)) rc = 4;
    if (rc == 0 && t.type == kTypeQ8_0) {
        const int64_t nb = static_cast<int64_t>(t.numel() / 32);
        if (scratch_dev) {
            // blocks as they are on disk -> device scratch, then one kernel splits them into the two planes
            if (cudaMemcpyAsync(scratch_dev, host, bytes, cudaMemcpyHostToDevice, st) != cudaSuccess) rc = 6;
            else rc = ppml_b200_repack_q8_0(scratch_dev, nb, dst_dev, st);
        } else {
            std::vector<uint8_t> planar(bytes);
            if (ppml_b200_repack_q8_0_host(host, nb, planar.data()) != 0) rc = 5;
            else {
                std::memcpy(host, planar.data(), bytes);
                if (cudaMemcpyAsync(dst_dev, host, bytes, cudaMemcpyHostToDevice, st) != cudaSuccess) rc = 6;
            }
        }
    } else if (rc == 0) {
        if (cudaMemcpyAsync(dst_dev, host, bytes, cudaMemcpyHostToDevice, st) != cudaSuccess) rc = 6;
    }
    if (cudaStreamSynchronize(st) != cudaSuccess && rc == 0) rc = 6;  // the pinned buffer is released below
    cudaFreeHost(host);
    if (rc == 6) cudaGetLastError();
    return rc;
}

}  // extern "C"
