// C wrapper around the REFERENCE's own artifact writer and reader, so that tests can cross-check this
// repository's reader and writer against them.  TEST INFRASTRUCTURE: it is compiled together with the
// reference's sources (src/artifact/{checksum,metadata,reader,writer}.cpp), from where they lie, into
// oracle/_ref/ by oracle/build.py when the reference tree is present; nothing of the reference is copied here.
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "reader.h"
#include "writer.h"

extern "C" {

// Writes an artifact with the reference's ArtifactWriter.  Returns 0 on success.
int ref_artifact_write(const char* path, const char* metadata_json, int n, const char* const* names, const uint32_t* types,
                       const void* const* datas, const uint64_t* sizes) {
    xinfer::artifact::ArtifactWriter w;
    if (metadata_json) w.set_raw_metadata_json(metadata_json);
    for (int i = 0; i < n; ++i)
        if (!w.add_section(names[i], static_cast<xinfer::artifact::SectionType>(types[i]), datas[i], static_cast<size_t>(sizes[i])))
            return 2;
    std::string err;
    return w.write_to_file(path, &err) ? 0 : 1;
}

// Opens with the reference's ArtifactReader, optionally validates the file checksum, reads one section.
// Returns the section's size (>= 0), -1 open failed, -2 checksum failed, -3 read failed, -4 buffer too small.
int64_t ref_artifact_read(const char* path, int validate, const char* name, void* dst, uint64_t capacity) {
    xinfer::artifact::ArtifactReader r;
    std::string err;
    if (!r.open(path, &err)) return -1;
    if (validate && !r.validate_checksum(&err)) return -2;
    if (!name) return 0;
    std::vector<uint8_t> data;
    if (!r.read_section(name, data, &err)) return -3;
    if (data.size() > capacity) return -4;
    if (!data.empty()) std::memcpy(dst, data.data(), data.size());
    return static_cast<int64_t>(data.size());
}

int ref_artifact_section_count(const char* path) {
    xinfer::artifact::ArtifactReader r;
    if (!r.open(path, nullptr)) return -1;
    return static_cast<int>(r.list_sections().size());
}

}  // extern "C"
