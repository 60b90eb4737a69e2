// Reading safetensors files: 8 bytes little-endian header length, a JSON header
// {name: {dtype, shape, data_offsets: [begin, end]}}, then the raw tensor bytes. The file is
// mapped read-only; every tensor is checked to lie inside the file and to hold as many bytes as
// its shape and dtype need, as the GGUF reader of MythEclipse/llm checks its tensors
// (apps/engine/src/gguf.rs:158-165). Callers read tensors straight from the map.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>

#include "json.hpp"

namespace llmh {

namespace {

struct DtypeWidth { const char* name; int bytes; };
const DtypeWidth DTYPES[] = {{"F64", 8}, {"F32", 4}, {"F16", 2}, {"BF16", 2}, {"I64", 8}, {"I32", 4},
                             {"I16", 2}, {"I8", 1},  {"U8", 1},  {"BOOL", 1}};
constexpr unsigned long long MAX_HEADER = 100ull << 20;

int width_of(const std::string& dtype) {
    for (const DtypeWidth& d : DTYPES)
        if (dtype == d.name) return d.bytes;
    return 0;
}

struct Entry {
    std::string name, dtype;
    std::vector<long long> shape;
    long long begin = 0, nbytes = 0;
};

}  // namespace

class SafetensorsFile {
public:
    explicit SafetensorsFile(const std::string& path) : path_(path) {
        fd_ = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
        if (fd_ < 0) throw Failure{LLMH_FORMAT, path + ": " + (errno == ENOENT ? "no such file" : std::strerror(errno))};
        struct stat st {};
        if (::fstat(fd_, &st) != 0 || !S_ISREG(st.st_mode)) fail_(LLMH_FORMAT, "no such file");
        size_ = (unsigned long long)st.st_size;
        if (size_ < 8) fail_(LLMH_FORMAT, "too short to be a safetensors file");
        map_ = ::mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
        if (map_ == MAP_FAILED) {
            map_ = nullptr;
            fail_(LLMH_IO, std::string("cannot be mapped: ") + std::strerror(errno));
        }
        const unsigned char* bytes = static_cast<const unsigned char*>(map_);
        unsigned long long header_len = 0;
        for (int i = 7; i >= 0; --i) header_len = (header_len << 8) | bytes[i];
        if (header_len > size_ - 8 || header_len > MAX_HEADER)
            fail_(LLMH_FORMAT, "header length " + std::to_string(header_len) + " exceeds the file");
        data_start_ = 8 + header_len;
        Json header;
        try {
            header = JsonReader(reinterpret_cast<const char*>(bytes + 8), header_len, path).read();
        } catch (const Failure& failure) {
            close_();
            throw Failure{LLMH_FORMAT, path_ + ": header is not JSON (" + failure.text + ")"};
        }
        if (header.kind != Json::Object) fail_(LLMH_FORMAT, "header is not an object");
        for (const auto& member : header.members) {
            if (member.first == "__metadata__") {
                if (member.second.kind == Json::Object)
                    for (const auto& item : member.second.members)
                        if (item.second.kind == Json::String) metadata_.emplace_back(item.first, item.second.string);
                continue;
            }
            entries_.push_back(entry_(member.first, member.second));
        }
    }
    ~SafetensorsFile() { close_(); }
    SafetensorsFile(const SafetensorsFile&) = delete;
    SafetensorsFile& operator=(const SafetensorsFile&) = delete;

    const std::vector<Entry>& entries() const { return entries_; }
    const std::vector<std::pair<std::string, std::string>>& metadata() const { return metadata_; }
    const unsigned char* data() const { return static_cast<const unsigned char*>(map_) + data_start_; }

private:
    std::string path_;
    int fd_ = -1;
    void* map_ = nullptr;
    unsigned long long size_ = 0, data_start_ = 0;
    std::vector<Entry> entries_;
    std::vector<std::pair<std::string, std::string>> metadata_;

    void close_() {
        if (map_) ::munmap(map_, size_);
        if (fd_ >= 0) ::close(fd_);
        map_ = nullptr;
        fd_ = -1;
    }
    [[noreturn]] void fail_(int code, const std::string& what) {
        close_();
        throw Failure{code, path_ + ": " + what};
    }
    Entry entry_(const std::string& name, const Json& value) {
        const Json* dtype = value.kind == Json::Object ? value.find("dtype") : nullptr;
        const Json* shape = value.kind == Json::Object ? value.find("shape") : nullptr;
        const Json* offsets = value.kind == Json::Object ? value.find("data_offsets") : nullptr;
        bool well_formed = dtype && dtype->kind == Json::String && shape && shape->kind == Json::Array && offsets &&
                           offsets->kind == Json::Array && offsets->items.size() == 2 &&
                           offsets->items[0].kind == Json::Integer && offsets->items[1].kind == Json::Integer;
        if (well_formed)
            for (const Json& d : shape->items) well_formed = well_formed && d.kind == Json::Integer && d.integer >= 0;
        if (!well_formed) fail_(LLMH_FORMAT, "malformed entry for '" + name + "'");
        Entry entry;
        entry.name = name;
        entry.dtype = dtype->string;
        int width = width_of(entry.dtype);
        if (!width) fail_(LLMH_FORMAT, "'" + name + "' has unknown dtype " + entry.dtype);
        unsigned __int128 count = 1;
        for (const Json& d : shape->items) {
            entry.shape.push_back(d.integer);
            count *= (unsigned long long)d.integer;
            if (count > (unsigned __int128)1 << 62) fail_(LLMH_FORMAT, "'" + name + "' has an impossible shape");
        }
        long long begin = offsets->items[0].integer, end = offsets->items[1].integer;
        if (begin < 0 || end < begin || data_start_ + (unsigned long long)end > size_)
            fail_(LLMH_FORMAT, "'" + name + "' lies outside the file");
        unsigned long long needed = (unsigned long long)count * width;
        if ((unsigned long long)(end - begin) != needed) {
            std::string dims;
            for (size_t i = 0; i < entry.shape.size(); ++i) dims += (i ? ", " : "") + std::to_string(entry.shape[i]);
            fail_(LLMH_FORMAT, "'" + name + "' holds " + std::to_string(end - begin) + " bytes, its shape [" + dims +
                                   "] needs " + std::to_string(needed));
        }
        entry.begin = begin;
        entry.nbytes = end - begin;
        return entry;
    }
};

}  // namespace llmh

using namespace llmh;

LLMH_EXPORT int llmh_safetensors_open(const char* path, void** out) {
    return guarded([&] { *out = new SafetensorsFile(path); });
}
LLMH_EXPORT void llmh_safetensors_close(void* file) { delete static_cast<SafetensorsFile*>(file); }
LLMH_EXPORT int llmh_safetensors_count(void* file) { return (int)static_cast<SafetensorsFile*>(file)->entries().size(); }
// Entry i: pointers stay valid until the file is closed. `address` is where its bytes are mapped.
LLMH_EXPORT int llmh_safetensors_entry(void* file, int i, const char** name, const char** dtype, int* rank,
                                       const long long** shape, const void** address, long long* nbytes) {
    return guarded([&] {
        const SafetensorsFile* f = static_cast<SafetensorsFile*>(file);
        if (i < 0 || i >= (int)f->entries().size()) throw Failure{LLMH_INVARIANT, "no such tensor entry"};
        const Entry& e = f->entries()[i];
        *name = e.name.c_str();
        *dtype = e.dtype.c_str();
        *rank = (int)e.shape.size();
        *shape = e.shape.data();
        *address = f->data() + e.begin;
        *nbytes = e.nbytes;
    });
}
LLMH_EXPORT int llmh_safetensors_metadata_count(void* file) { return (int)static_cast<SafetensorsFile*>(file)->metadata().size(); }
LLMH_EXPORT int llmh_safetensors_metadata_item(void* file, int i, const char** key, const char** value) {
    return guarded([&] {
        const SafetensorsFile* f = static_cast<SafetensorsFile*>(file);
        if (i < 0 || i >= (int)f->metadata().size()) throw Failure{LLMH_INVARIANT, "no such metadata item"};
        *key = f->metadata()[i].first.c_str();
        *value = f->metadata()[i].second.c_str();
    });
}
