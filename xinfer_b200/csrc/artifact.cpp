// Reader of `.xinfer` artifacts and loader of their INT4 tensors into device memory, N-sharded on request.
//
// What it stands in for in the reference:
//   container layout (header, section table, footer)      src/artifact/container.h:20-63, docs/artifact-format.md
//   ArtifactReader::open / read_section / validate_checksum   src/artifact/reader.cpp:59-310
//   load_linear (size checks of an INT4 projection)       src/targets/qwen3_8_27b/weights.cpp:252-304
//   load_bf16_as_fp32 (norm weights, the 1 + w convention)   src/targets/qwen3_8_27b/weights.cpp:319-347
// Differences: sections stream from the file through pinned staging buffers straight into device memory (the
// reference reads a whole section into a std::vector first); a projection can be loaded as a row range
// [row0, row0 + rows) of W_int4 / scales, which is the N-split shard of a tensor-parallel rank and needs no
// re-packing because both tensors are row-major over output features; the CRC-64 of a section is computed
// while it streams (always over the whole section, also when only a row range is kept).
#include <cuda_runtime.h>
#include <fcntl.h>
#include <stdint.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#include <new>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/xinfer_b200.h"
#include "w4a16.h"

namespace {

#pragma pack(push, 1)
struct Header {  // 64 bytes
    uint8_t magic[8];
    uint32_t format_version, header_size, flags, section_count;
    uint64_t metadata_offset, metadata_size, section_table_offset, section_table_size, total_file_size;
};
struct Entry {  // 128 bytes
    char name[96];
    uint32_t type_tag, flags;
    uint64_t offset, size, checksum;
};
struct Footer {  // 16 bytes
    uint64_t file_checksum;
    uint8_t magic[8];
};
#pragma pack(pop)
static_assert(sizeof(Header) == 64 && sizeof(Entry) == 128 && sizeof(Footer) == 16, "container records");

const uint8_t kMagic[8] = {'X', 'I', 'N', 'F', 'E', 'R', 0, 0};
const uint8_t kFooterMagic[8] = {'X', 'I', 'N', 'F', 'F', 'O', 'O', 'T'};
constexpr size_t kChunk = 8u << 20;  // streaming granularity: two pinned buffers of this size

bool pread_all(int fd, void* dst, size_t n, uint64_t off) {
    uint8_t* p = static_cast<uint8_t*>(dst);
    while (n > 0) {
        const ssize_t got = pread(fd, p, n, static_cast<off_t>(off));
        if (got <= 0) return false;
        p += got;
        off += static_cast<uint64_t>(got);
        n -= static_cast<size_t>(got);
    }
    return true;
}

}  // namespace

struct xinfer_artifact {
    int fd = -1;
    uint64_t file_size = 0;
    Header header{};
    Footer footer{};
    std::vector<Entry> sections;
    std::unordered_map<std::string, int> index;
    std::string metadata, error;
    uint8_t* stage[2] = {nullptr, nullptr};  // pinned
    cudaEvent_t stage_free[2] = {nullptr, nullptr};
    cudaStream_t stream = nullptr;
};

namespace {

int fail(xinfer_artifact* a, int code, const std::string& msg) {
    if (a) a->error = msg;
    xb::set_last_error(msg.c_str());
    return code;
}

bool ensure_staging(xinfer_artifact* a) {
    if (a->stage[0]) return true;
    if (cudaStreamCreateWithFlags(&a->stream, cudaStreamNonBlocking) != cudaSuccess) return false;
    for (int i = 0; i < 2; ++i) {
        if (cudaMallocHost(reinterpret_cast<void**>(&a->stage[i]), kChunk) != cudaSuccess) return false;
        if (cudaEventCreateWithFlags(&a->stage_free[i], cudaEventDisableTiming) != cudaSuccess) return false;
    }
    return true;
}

// Streams section `e` from the file; the bytes [keep_off, keep_off + keep_len) of it go to `dst_dev` (device) or
// `dst_host`.  Returns the CRC-64 of the WHOLE section through *crc_out when `want_crc`.
int stream_section(xinfer_artifact* a, const Entry& e, uint64_t keep_off, uint64_t keep_len, void* dst_dev, void* dst_host,
                   bool want_crc, uint64_t* crc_out) {
    if (keep_off + keep_len > e.size) return fail(a, XINFER_ERR_INVALID_ARGUMENT, "range outside the section");
    if (dst_dev && !ensure_staging(a)) return fail(a, XINFER_ERR_OUT_OF_MEMORY, "pinned staging buffers");
    std::vector<uint8_t> host_tmp;
    if (!dst_dev) host_tmp.resize(kChunk);
    // without a CRC only the kept range is read
    uint64_t pos = want_crc ? 0 : keep_off;
    const uint64_t end = want_crc ? e.size : keep_off + keep_len;
    int slot = 0;
    uint64_t running = ~0ull;  // CRC-64 state: all ones going in, complemented coming out
    while (pos < end) {
        const size_t n = static_cast<size_t>(end - pos < kChunk ? end - pos : kChunk);
        uint8_t* buf;
        if (dst_dev) {
            buf = a->stage[slot];
            if (cudaEventSynchronize(a->stage_free[slot]) != cudaSuccess) return fail(a, XINFER_ERR_CUDA, "staging event");
        } else {
            buf = host_tmp.data();
        }
        if (!pread_all(a->fd, buf, n, e.offset + pos)) return fail(a, XINFER_ERR_INVALID_ARGUMENT, std::string("short read in section ") + e.name);
        if (want_crc) running = xinfer_crc64_update(running, buf, n);
        // the part of this chunk that is kept
        const uint64_t lo = pos > keep_off ? pos : keep_off;
        const uint64_t hi = (pos + n) < (keep_off + keep_len) ? (pos + n) : (keep_off + keep_len);
        if (hi > lo) {
            if (dst_dev) {
                if (cudaMemcpyAsync(static_cast<uint8_t*>(dst_dev) + (lo - keep_off), buf + (lo - pos), hi - lo, cudaMemcpyHostToDevice,
                                    a->stream) != cudaSuccess)
                    return fail(a, XINFER_ERR_CUDA, "copy to device");
                cudaEventRecord(a->stage_free[slot], a->stream);
                slot ^= 1;
            } else if (dst_host) {
                memcpy(static_cast<uint8_t*>(dst_host) + (lo - keep_off), buf + (lo - pos), hi - lo);
            }
        }
        pos += n;
    }
    if (dst_dev && cudaStreamSynchronize(a->stream) != cudaSuccess) return fail(a, XINFER_ERR_CUDA, "copy to device");
    if (want_crc && crc_out) *crc_out = ~running;
    return XINFER_OK;
}

}  // namespace

extern "C" {

int xinfer_artifact_open(const char* path, int verify_file_checksum, xinfer_artifact** out) {
    if (!path || !out) return XINFER_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    xinfer_artifact* a = new (std::nothrow) xinfer_artifact();
    if (!a) return XINFER_ERR_OUT_OF_MEMORY;
    auto bad = [&](const std::string& msg) {
        fail(nullptr, XINFER_ERR_INVALID_ARGUMENT, msg);
        xinfer_artifact_close(a);
        return XINFER_ERR_INVALID_ARGUMENT;
    };
    a->fd = open(path, O_RDONLY);
    if (a->fd < 0) return bad(std::string("could not open file: ") + path);
    struct stat st;
    if (fstat(a->fd, &st) != 0) return bad("could not stat the file");
    a->file_size = static_cast<uint64_t>(st.st_size);
    if (a->file_size < sizeof(Header) + sizeof(Footer)) return bad("file is smaller than header plus footer");
    if (!pread_all(a->fd, &a->header, sizeof(Header), 0)) return bad("failed to read the header");
    const Header& h = a->header;
    if (memcmp(h.magic, kMagic, 8) != 0) return bad("invalid file magic; not a .xinfer artifact");
    if (h.format_version != 1) return bad("unsupported .xinfer format version " + std::to_string(h.format_version));
    if (h.header_size != sizeof(Header)) return bad("corrupted header size field");
    if (h.total_file_size != a->file_size) return bad("file size mismatch: header expects " + std::to_string(h.total_file_size) +
                                                      " bytes, file has " + std::to_string(a->file_size));
    if (!pread_all(a->fd, &a->footer, sizeof(Footer), a->file_size - sizeof(Footer))) return bad("failed to read the footer");
    if (memcmp(a->footer.magic, kFooterMagic, 8) != 0) return bad("invalid footer magic; file may be corrupted or truncated");
    if (h.metadata_size > 0) {
        if (h.metadata_offset + h.metadata_size > a->file_size || h.metadata_offset + h.metadata_size < h.metadata_offset)
            return bad("metadata block points out of bounds");
        a->metadata.resize(h.metadata_size);
        if (!pread_all(a->fd, &a->metadata[0], h.metadata_size, h.metadata_offset)) return bad("failed to read the metadata block");
    }
    if (h.section_count > 0) {
        const uint64_t table = static_cast<uint64_t>(h.section_count) * sizeof(Entry);
        if (h.section_table_size != table) return bad("section table size does not match the section count");
        if (h.section_table_offset + table > a->file_size) return bad("section table points out of bounds");
        a->sections.resize(h.section_count);
        if (!pread_all(a->fd, a->sections.data(), table, h.section_table_offset)) return bad("failed to read the section table");
        for (size_t i = 0; i < a->sections.size(); ++i) {
            Entry& e = a->sections[i];
            e.name[sizeof(e.name) - 1] = 0;
            if (e.offset + e.size > a->file_size || e.offset + e.size < e.offset)
                return bad(std::string("section '") + e.name + "' points out of bounds");
            a->index[e.name] = static_cast<int>(i);
        }
    }
    if (verify_file_checksum) {
        // CRC-64 of every byte before the footer, src/artifact/reader.cpp:266-310
        uint64_t running = ~0ull;
        std::vector<uint8_t> buf(kChunk);
        const uint64_t end = a->file_size - sizeof(Footer);
        for (uint64_t pos = 0; pos < end;) {
            const size_t n = static_cast<size_t>(end - pos < kChunk ? end - pos : kChunk);
            if (!pread_all(a->fd, buf.data(), n, pos)) return bad("short read while checking the file checksum");
            running = xinfer_crc64_update(running, buf.data(), n);
            pos += n;
        }
        if (~running != a->footer.file_checksum) return bad("file checksum mismatch");
    }
    *out = a;
    return XINFER_OK;
}

void xinfer_artifact_close(xinfer_artifact* a) {
    if (!a) return;
    if (a->fd >= 0) close(a->fd);
    for (int i = 0; i < 2; ++i) {
        if (a->stage[i]) cudaFreeHost(a->stage[i]);
        if (a->stage_free[i]) cudaEventDestroy(a->stage_free[i]);
    }
    if (a->stream) cudaStreamDestroy(a->stream);
    delete a;
}

int xinfer_artifact_section_count(const xinfer_artifact* a) { return a ? static_cast<int>(a->sections.size()) : 0; }

int xinfer_artifact_find(const xinfer_artifact* a, const char* name) {
    if (!a || !name) return -1;
    auto it = a->index.find(name);
    return it == a->index.end() ? -1 : it->second;
}

int xinfer_artifact_section_info(const xinfer_artifact* a, int index, const char** name, uint32_t* type_tag, uint64_t* offset,
                                 uint64_t* size, uint64_t* checksum) {
    if (!a || index < 0 || index >= static_cast<int>(a->sections.size())) return XINFER_ERR_INVALID_ARGUMENT;
    const Entry& e = a->sections[index];
    if (name) *name = e.name;
    if (type_tag) *type_tag = e.type_tag;
    if (offset) *offset = e.offset;
    if (size) *size = e.size;
    if (checksum) *checksum = e.checksum;
    return XINFER_OK;
}

const char* xinfer_artifact_metadata(const xinfer_artifact* a, uint64_t* size) {
    if (!a) return nullptr;
    if (size) *size = a->metadata.size();
    return a->metadata.c_str();
}

const char* xinfer_artifact_error(const xinfer_artifact* a) { return a ? a->error.c_str() : ""; }

int xinfer_artifact_read_section(xinfer_artifact* a, const char* name, void* dst_host, uint64_t capacity) {
    const int i = xinfer_artifact_find(a, name);
    if (i < 0) return fail(a, XINFER_ERR_INVALID_ARGUMENT, std::string("section not found: ") + (name ? name : ""));
    const Entry& e = a->sections[i];
    if (!dst_host || capacity < e.size) return fail(a, XINFER_ERR_INVALID_ARGUMENT, "destination smaller than the section");
    uint64_t crc = 0;
    int rc = stream_section(a, e, 0, e.size, nullptr, dst_host, true, &crc);
    if (rc != XINFER_OK) return rc;
    if (crc != e.checksum) return fail(a, XINFER_ERR_CONTRACT, std::string("checksum mismatch in section ") + e.name);
    return XINFER_OK;
}

int xinfer_artifact_load_section(xinfer_artifact* a, const char* name, uint64_t offset, uint64_t bytes, void* dst_dev, int verify) {
    const int i = xinfer_artifact_find(a, name);
    if (i < 0) return fail(a, XINFER_ERR_INVALID_ARGUMENT, std::string("section not found: ") + (name ? name : ""));
    const Entry& e = a->sections[i];
    if (!dst_dev) return fail(a, XINFER_ERR_INVALID_ARGUMENT, "null destination");
    uint64_t crc = 0;
    int rc = stream_section(a, e, offset, bytes, dst_dev, nullptr, verify != 0, &crc);
    if (rc != XINFER_OK) return rc;
    if (verify && crc != e.checksum) return fail(a, XINFER_ERR_CONTRACT, std::string("checksum mismatch in section ") + e.name);
    return XINFER_OK;
}

int xinfer_artifact_load_linear(xinfer_artifact* a, const char* weight_name, int64_t out_features, int64_t in_features,
                                int group_size, int64_t row0, int64_t rows, void* dst_weights_dev, void* dst_scales_dev,
                                int verify) {
    if (!a || !weight_name || out_features <= 0 || in_features <= 0 || group_size <= 0 || in_features % 2 ||
        row0 < 0 || rows <= 0 || row0 + rows > out_features)
        return fail(a, XINFER_ERR_INVALID_ARGUMENT, "load_linear: bad shape or row range");
    const std::string wn(weight_name), sn = wn + ".scales";  // src/targets/qwen3_8_27b/weights.cpp:284
    const int wi = xinfer_artifact_find(a, wn.c_str()), si = xinfer_artifact_find(a, sn.c_str());
    if (wi < 0) return fail(a, XINFER_ERR_INVALID_ARGUMENT, "section not found: " + wn);
    if (si < 0) return fail(a, XINFER_ERR_INVALID_ARGUMENT, "section not found: " + sn);
    const uint64_t w_row = static_cast<uint64_t>(in_features / 2), s_row = static_cast<uint64_t>(in_features / group_size) * 2;
    const uint64_t want_w = static_cast<uint64_t>(out_features) * w_row, want_s = static_cast<uint64_t>(out_features) * s_row;
    if (a->sections[wi].size != want_w)
        return fail(a, XINFER_ERR_INVALID_ARGUMENT, "weight size mismatch for " + wn + ": expected " + std::to_string(want_w) +
                                                        ", got " + std::to_string(a->sections[wi].size));
    if (a->sections[si].size != want_s)
        return fail(a, XINFER_ERR_INVALID_ARGUMENT, "scales size mismatch for " + sn + ": expected " + std::to_string(want_s) +
                                                        ", got " + std::to_string(a->sections[si].size));
    int rc = xinfer_artifact_load_section(a, wn.c_str(), static_cast<uint64_t>(row0) * w_row, static_cast<uint64_t>(rows) * w_row,
                                          dst_weights_dev, verify);
    if (rc != XINFER_OK) return rc;
    return xinfer_artifact_load_section(a, sn.c_str(), static_cast<uint64_t>(row0) * s_row, static_cast<uint64_t>(rows) * s_row,
                                        dst_scales_dev, verify);
}

int xinfer_artifact_load_bf16_as_f32(xinfer_artifact* a, const char* name, int64_t num_elements, int add_unit_offset,
                                     float* dst_dev) {
    const int i = xinfer_artifact_find(a, name);
    if (i < 0) return fail(a, XINFER_ERR_INVALID_ARGUMENT, std::string("section not found: ") + (name ? name : ""));
    const Entry& e = a->sections[i];
    if (num_elements <= 0 || !dst_dev) return fail(a, XINFER_ERR_INVALID_ARGUMENT, "load_bf16_as_f32: bad arguments");
    if (e.size != static_cast<uint64_t>(num_elements) * 2)
        return fail(a, XINFER_ERR_INVALID_ARGUMENT, std::string("element count mismatch for ") + e.name + ": expected " +
                                                        std::to_string(num_elements * 2) + " bytes, got " + std::to_string(e.size));
    std::vector<uint16_t> raw(static_cast<size_t>(num_elements));
    uint64_t crc = 0;
    int rc = stream_section(a, e, 0, e.size, nullptr, raw.data(), true, &crc);
    if (rc != XINFER_OK) return rc;
    if (crc != e.checksum) return fail(a, XINFER_ERR_CONTRACT, std::string("checksum mismatch in section ") + e.name);
    std::vector<float> f(raw.size());
    for (size_t j = 0; j < raw.size(); ++j) {
        const uint32_t bits = static_cast<uint32_t>(raw[j]) << 16;
        float v;
        memcpy(&v, &bits, 4);
        f[j] = add_unit_offset ? v + 1.0f : v;  // Qwen's RMSNorm stores w - 1, src/targets/qwen3_8_27b/weights.cpp:319-347
    }
    if (cudaMemcpy(dst_dev, f.data(), f.size() * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess)
        return fail(a, XINFER_ERR_CUDA, "copy to device");
    return XINFER_OK;
}

}  // extern "C"
