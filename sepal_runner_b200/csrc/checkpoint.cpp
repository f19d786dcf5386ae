#include "checkpoint.hpp"

#include <algorithm>
#include <cerrno>
#include <cstdio>
#include <cstring>
#include <filesystem>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace sepal::b200 {

namespace {

struct TypeRow {
    ElementType type;
    const char* name;
    std::size_t bytes;
};
constexpr TypeRow kTypes[] = {
    {ElementType::F32, "F32", 4}, {ElementType::F16, "F16", 2}, {ElementType::BF16, "BF16", 2}, {ElementType::I8, "I8", 1},  {ElementType::U8, "U8", 1},
    {ElementType::I32, "I32", 4}, {ElementType::I64, "I64", 8}, {ElementType::F64, "F64", 8},   {ElementType::Bool, "BOOL", 1}, {ElementType::I16, "I16", 2},
    {ElementType::U16, "U16", 2}, {ElementType::U32, "U32", 4}, {ElementType::U64, "U64", 8},
};

// The header is one JSON object whose members are objects of strings, numbers and arrays of numbers; "__metadata__" maps strings to
// strings. The scanner below reads exactly that much JSON (strings with the standard escapes, non-negative integers, nesting) and
// refuses anything else.
class HeaderScanner {
public:
    HeaderScanner(const char* text, std::size_t size, const std::string& origin) : p_(text), end_(text + size), origin_(origin) {}

    [[noreturn]] void fail(const std::string& what) const { throw CheckpointError(origin_ + ": malformed header: " + what); }
    void skip_space() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\t' || *p_ == '\n' || *p_ == '\r')) ++p_;
    }
    bool peek(char c) {
        skip_space();
        return p_ < end_ && *p_ == c;
    }
    void expect(char c) {
        skip_space();
        if (p_ >= end_ || *p_ != c) fail(std::string("expected '") + c + "'");
        ++p_;
    }
    bool at_end() {
        skip_space();
        return p_ >= end_;
    }
    std::string string() {
        expect('"');
        std::string out;
        while (true) {
            if (p_ >= end_) fail("unterminated string");
            const char c = *p_++;
            if (c == '"') return out;
            if (static_cast<unsigned char>(c) < 0x20) fail("control character in a string");
            if (c != '\\') {
                out.push_back(c);
                continue;
            }
            if (p_ >= end_) fail("unterminated escape");
            const char e = *p_++;
            switch (e) {
            case '"': out.push_back('"'); break;
            case '\\': out.push_back('\\'); break;
            case '/': out.push_back('/'); break;
            case 'b': out.push_back('\b'); break;
            case 'f': out.push_back('\f'); break;
            case 'n': out.push_back('\n'); break;
            case 'r': out.push_back('\r'); break;
            case 't': out.push_back('\t'); break;
            case 'u': {
                if (end_ - p_ < 4) fail("short \\u escape");
                unsigned code = 0;
                for (int i = 0; i < 4; ++i) {
                    const char h = *p_++;
                    code <<= 4;
                    if (h >= '0' && h <= '9') code |= static_cast<unsigned>(h - '0');
                    else if (h >= 'a' && h <= 'f') code |= static_cast<unsigned>(h - 'a' + 10);
                    else if (h >= 'A' && h <= 'F') code |= static_cast<unsigned>(h - 'A' + 10);
                    else fail("bad \\u escape");
                }
                // UTF-8 of a code point of the basic plane (surrogate pairs do not occur in tensor names; kept as they are encoded)
                if (code < 0x80) out.push_back(static_cast<char>(code));
                else if (code < 0x800) {
                    out.push_back(static_cast<char>(0xC0 | (code >> 6)));
                    out.push_back(static_cast<char>(0x80 | (code & 0x3F)));
                } else {
                    out.push_back(static_cast<char>(0xE0 | (code >> 12)));
                    out.push_back(static_cast<char>(0x80 | ((code >> 6) & 0x3F)));
                    out.push_back(static_cast<char>(0x80 | (code & 0x3F)));
                }
                break;
            }
            default: fail("unknown escape");
            }
        }
    }
    std::uint64_t number() {
        skip_space();
        if (p_ >= end_ || *p_ < '0' || *p_ > '9') fail("expected a non-negative whole number");
        std::uint64_t v = 0;
        while (p_ < end_ && *p_ >= '0' && *p_ <= '9') {
            const std::uint64_t digit = static_cast<std::uint64_t>(*p_ - '0');
            if (v > (UINT64_MAX - digit) / 10) fail("number too large");
            v = v * 10 + digit;
            ++p_;
        }
        if (p_ < end_ && (*p_ == '.' || *p_ == 'e' || *p_ == 'E' || *p_ == '-')) fail("expected a whole number");
        return v;
    }
    std::vector<std::uint64_t> numbers() {
        std::vector<std::uint64_t> out;
        expect('[');
        if (peek(']')) {
            ++p_;
            return out;
        }
        while (true) {
            out.push_back(number());
            if (peek(',')) {
                ++p_;
                continue;
            }
            expect(']');
            return out;
        }
    }

private:
    const char* p_;
    const char* end_;
    const std::string& origin_;
};

std::uint64_t checked_product(const std::vector<std::uint64_t>& shape, const std::string& where) {
    std::uint64_t n = 1;
    for (const std::uint64_t d : shape) {
        if (d != 0 && n > UINT64_MAX / d) throw CheckpointError(where + ": the shape overflows");
        n *= d;
    }
    return n;
}

}  // namespace

std::size_t bytes_of(ElementType type) {
    for (const TypeRow& r : kTypes)
        if (r.type == type) return r.bytes;
    return 0;
}
const char* name_of(ElementType type) {
    for (const TypeRow& r : kTypes)
        if (r.type == type) return r.name;
    return "?";
}

std::uint64_t TensorView::elements() const {
    std::uint64_t n = 1;
    for (const std::uint64_t d : shape) n *= d;
    return n;
}

TensorFile::~TensorFile() {
    if (mapping_ != nullptr) (void)munmap(mapping_, mapped_bytes_);
}

std::shared_ptr<const TensorFile> TensorFile::open(const std::string& path) {
    const int fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
    if (fd < 0) throw std::runtime_error(path + ": cannot open: " + std::strerror(errno));
    struct stat st {};
    if (fstat(fd, &st) != 0 || !S_ISREG(st.st_mode)) {
        (void)close(fd);
        throw std::runtime_error(path + ": not a regular file");
    }
    const std::size_t size = static_cast<std::size_t>(st.st_size);
    if (size < 8) {
        (void)close(fd);
        throw CheckpointError(path + ": shorter than the 8-byte header length");
    }
    void* map = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
    (void)close(fd);
    if (map == MAP_FAILED) throw std::runtime_error(path + ": cannot map: " + std::strerror(errno));
    std::shared_ptr<TensorFile> file(new TensorFile());
    file->mapping_ = map;
    file->mapped_bytes_ = size;
    file->origin_ = path;
    file->parse(static_cast<const unsigned char*>(map), size);
    return file;
}

std::shared_ptr<const TensorFile> TensorFile::from_memory(const unsigned char* bytes, std::size_t size, std::string origin) {
    std::shared_ptr<TensorFile> file(new TensorFile());
    file->origin_ = std::move(origin);
    if (bytes == nullptr || size < 8) throw CheckpointError(file->origin_ + ": shorter than the 8-byte header length");
    file->parse(bytes, size);
    return file;
}

void TensorFile::parse(const unsigned char* bytes, std::size_t size) {
    std::uint64_t header_bytes = 0;
    for (int i = 7; i >= 0; --i) header_bytes = (header_bytes << 8) | bytes[i];
    // The limits the reference's reader sets (runner/src/io/safetensors.cpp:21-23,131-248): a header above 100 MB is a damaged or hostile
    // file; so is a rank above 32. (The tensor descriptions of this library's own C ABI stop at rank 8, far above any weight's.)
    constexpr std::uint64_t kMaxHeaderBytes = 100'000'000;
    constexpr std::size_t kMaxRank = 32;
    if (header_bytes > kMaxHeaderBytes) throw CheckpointError(origin_ + ": the header claims " + std::to_string(header_bytes) + " bytes, above the limit of 100 MB");
    if (header_bytes > size - 8) throw CheckpointError(origin_ + ": the header length " + std::to_string(header_bytes) + " is past the end of the file");
    if (header_bytes < 2) throw CheckpointError(origin_ + ": the header is empty");
    const unsigned char* data = bytes + 8 + header_bytes;
    const std::uint64_t data_bytes = size - 8 - header_bytes;

    HeaderScanner scan(reinterpret_cast<const char*>(bytes + 8), header_bytes, origin_);
    scan.expect('{');
    bool first = true, seen_metadata = false;
    while (!scan.peek('}')) {
        if (!first) scan.expect(',');
        first = false;
        const std::string name = scan.string();
        scan.expect(':');
        scan.expect('{');
        if (name == "__metadata__") {
            if (seen_metadata) throw CheckpointError(origin_ + ": '__metadata__' appears twice");
            seen_metadata = true;
            bool first_meta = true;
            while (!scan.peek('}')) {
                if (!first_meta) scan.expect(',');
                first_meta = false;
                const std::string key = scan.string();
                scan.expect(':');
                metadata_[key] = scan.string();
            }
            scan.expect('}');
            continue;
        }
        TensorView t;
        t.name = name;
        bool has_type = false, has_shape = false, has_offsets = false;
        std::vector<std::uint64_t> offsets;
        bool first_member = true;
        while (!scan.peek('}')) {
            if (!first_member) scan.expect(',');
            first_member = false;
            const std::string key = scan.string();
            scan.expect(':');
            if (key == "dtype") {
                const std::string type = scan.string();
                bool known = false;
                for (const TypeRow& r : kTypes)
                    if (type == r.name) {
                        t.type = r.type;
                        known = true;
                    }
                if (!known) throw CheckpointError(origin_ + ": tensor '" + name + "' has the unknown element type '" + type + "'");
                has_type = true;
            } else if (key == "shape") {
                t.shape = scan.numbers();
                if (t.shape.size() > kMaxRank) throw CheckpointError(origin_ + ": tensor '" + name + "' has rank " + std::to_string(t.shape.size()) + ", above the limit of 32");
                has_shape = true;
            } else if (key == "data_offsets") {
                offsets = scan.numbers();
                has_offsets = true;
            } else {
                throw CheckpointError(origin_ + ": tensor '" + name + "' has the unknown member '" + key + "'");
            }
        }
        scan.expect('}');
        if (!has_type || !has_shape || !has_offsets) throw CheckpointError(origin_ + ": tensor '" + name + "' lacks dtype, shape or data_offsets");
        if (offsets.size() != 2 || offsets[0] > offsets[1]) throw CheckpointError(origin_ + ": tensor '" + name + "' has malformed data_offsets");
        if (offsets[1] > data_bytes) throw CheckpointError(origin_ + ": tensor '" + name + "' ends past the end of the file");
        const std::uint64_t elements = checked_product(t.shape, origin_ + ": tensor '" + name + "'");
        const std::uint64_t width = bytes_of(t.type);
        if (elements > UINT64_MAX / width || elements * width != offsets[1] - offsets[0])
            throw CheckpointError(origin_ + ": tensor '" + name + "' holds " + std::to_string(offsets[1] - offsets[0]) + " bytes, its shape and type need " +
                                  std::to_string(elements * width));
        t.data = data + offsets[0];
        t.bytes = offsets[1] - offsets[0];
        if (t.bytes != 0 && reinterpret_cast<std::uintptr_t>(t.data) % width != 0)
            throw CheckpointError(origin_ + ": tensor '" + name + "' is not aligned for its " + std::to_string(width) + "-byte elements");
        if (index_.count(name) != 0) throw CheckpointError(origin_ + ": tensor '" + name + "' appears twice");
        index_[name] = tensors_.size();
        tensors_.push_back(std::move(t));
    }
    scan.expect('}');
    if (!scan.at_end()) scan.fail("text after the header object");

    // File order (empty tensors before a non-empty one that starts at the same byte), then one walk over the data section: every byte must
    // belong to exactly one tensor, so a tensor that starts before the bytes covered so far overlaps an earlier one, one that starts
    // after them leaves a hole, and what is left behind the last one belongs to nobody. The format asks for exactly this.
    std::sort(tensors_.begin(), tensors_.end(), [](const TensorView& a, const TensorView& b) { return a.data != b.data ? a.data < b.data : a.bytes < b.bytes; });
    std::uint64_t covered = 0;
    for (std::size_t i = 0; i < tensors_.size(); ++i) {
        index_[tensors_[i].name] = i;
        const std::uint64_t begin = static_cast<std::uint64_t>(tensors_[i].data - data);
        if (begin < covered) throw CheckpointError(origin_ + ": tensor '" + tensors_[i].name + "' overlaps the bytes of a tensor before it");
        if (begin > covered)
            throw CheckpointError(origin_ + ": bytes " + std::to_string(covered) + " to " + std::to_string(begin) + " of the data, before tensor '" + tensors_[i].name +
                                  "', belong to no tensor");
        covered = begin + tensors_[i].bytes;
    }
    if (covered != data_bytes) throw CheckpointError(origin_ + ": the last " + std::to_string(data_bytes - covered) + " bytes of the file belong to no tensor");
}

const TensorView* TensorFile::find(std::string_view name) const {
    const auto it = index_.find(name);
    return it == index_.end() ? nullptr : &tensors_[it->second];
}

std::shared_ptr<const Checkpoint> Checkpoint::from_files(std::vector<std::shared_ptr<const TensorFile>> files) {
    std::shared_ptr<Checkpoint> c(new Checkpoint());
    c->files_ = std::move(files);
    for (const auto& file : c->files_) {
        for (const TensorView& t : file->tensors()) {
            const auto [it, fresh] = c->by_name_.emplace(t.name, &t);
            if (!fresh) throw CheckpointError(file->origin() + ": tensor '" + t.name + "' is also in another file of the checkpoint");
        }
    }
    static constexpr std::string_view kPrefixes[] = {"model.language_model.", "language_model.", "model.", ""};
    bool found = false;
    for (const std::string_view prefix : kPrefixes) {
        if (c->by_name_.find(std::string(prefix) + "embed_tokens.weight") != c->by_name_.end()) {
            c->prefix_ = std::string(prefix);
            found = true;
            break;
        }
    }
    if (!found) c->prefix_.clear();  // a file of placed weights, or of anything else: names are used as they are
    return c;
}

std::shared_ptr<const Checkpoint> Checkpoint::open(const std::string& path) {
    namespace fs = std::filesystem;
    std::vector<std::shared_ptr<const TensorFile>> files;
    std::error_code ec;
    if (fs::is_regular_file(path, ec)) {
        files.push_back(TensorFile::open(path));
        return from_files(std::move(files));
    }
    if (!fs::is_directory(path, ec)) throw std::runtime_error(path + ": neither a file nor a directory");
    const fs::path single = fs::path(path) / "model.safetensors";
    if (fs::is_regular_file(single, ec)) {
        files.push_back(TensorFile::open(single.string()));
        return from_files(std::move(files));
    }
    // Shards model-0000i-of-0000N.safetensors: all N of one N.
    std::map<unsigned, std::map<unsigned, std::string>> shards;  // N -> i -> path
    for (const fs::directory_entry& entry : fs::directory_iterator(path)) {
        const std::string file = entry.path().filename().string();
        unsigned i = 0, n = 0;
        char tail[32] = {};
        if (std::sscanf(file.c_str(), "model-%5u-of-%5u.%31s", &i, &n, tail) == 3 && std::string(tail) == "safetensors" && file.size() == 32) shards[n][i] = entry.path().string();
    }
    if (shards.empty()) throw std::runtime_error(path + ": holds neither model.safetensors nor shards model-0000i-of-0000N.safetensors");
    if (shards.size() != 1) throw CheckpointError(path + ": holds shards of more than one checkpoint");
    const auto& [n, parts] = *shards.begin();
    for (unsigned i = 1; i <= n; ++i) {
        const auto it = parts.find(i);
        if (it == parts.end()) throw CheckpointError(path + ": shard " + std::to_string(i) + " of " + std::to_string(n) + " is missing");
        files.push_back(TensorFile::open(it->second));
    }
    if (parts.size() != n) throw CheckpointError(path + ": holds shards numbered outside 1 .. " + std::to_string(n));
    return from_files(std::move(files));
}

const TensorView* Checkpoint::find(std::string_view engine_name) const {
    const auto it = by_name_.find(prefix_ + std::string(engine_name));
    return it == by_name_.end() ? nullptr : it->second;
}

const TensorView& Checkpoint::at(std::string_view engine_name) const {
    const TensorView* t = find(engine_name);
    if (t == nullptr) throw std::out_of_range("the checkpoint has no tensor '" + prefix_ + std::string(engine_name) + "'");
    return *t;
}

std::vector<std::string> Checkpoint::names() const {
    std::vector<std::string> out;
    for (const auto& [name, view] : by_name_) {
        (void)view;
        if (name.compare(0, prefix_.size(), prefix_) == 0) out.push_back(name.substr(prefix_.size()));
    }
    return out;
}

std::string Checkpoint::metadata(std::string_view key) const {
    for (const auto& file : files_) {
        const auto it = file->metadata().find(key);
        if (it != file->metadata().end()) return it->second;
    }
    return {};
}

void write_tensor_file(const std::string& path, const std::vector<TensorToWrite>& tensors, const std::map<std::string, std::string>& metadata) {
    const auto quoted = [](const std::string& s) {
        std::string out = "\"";
        for (const char c : s) {
            if (c == '"' || c == '\\') {
                out.push_back('\\');
                out.push_back(c);
            } else if (static_cast<unsigned char>(c) < 0x20) {
                char buf[8];
                std::snprintf(buf, sizeof buf, "\\u%04x", static_cast<unsigned>(static_cast<unsigned char>(c)));
                out += buf;
            } else {
                out.push_back(c);
            }
        }
        out.push_back('"');
        return out;
    };
    std::string header = "{";
    if (!metadata.empty()) {
        header += "\"__metadata__\":{";
        bool first = true;
        for (const auto& [key, value] : metadata) {
            if (!first) header += ",";
            first = false;
            header += quoted(key) + ":" + quoted(value);
        }
        header += "},";
    }
    std::uint64_t at = 0;
    for (std::size_t i = 0; i < tensors.size(); ++i) {
        const TensorToWrite& t = tensors[i];
        std::uint64_t elements = 1;
        for (const std::uint64_t d : t.shape) elements *= d;
        const std::uint64_t bytes = elements * bytes_of(t.type);
        if (i != 0) header += ",";
        header += quoted(t.name) + ":{\"dtype\":\"" + name_of(t.type) + "\",\"shape\":[";
        for (std::size_t d = 0; d < t.shape.size(); ++d) header += (d ? "," : "") + std::to_string(t.shape[d]);
        header += "],\"data_offsets\":[" + std::to_string(at) + "," + std::to_string(at + bytes) + "]}";
        at += bytes;
    }
    header += "}";
    while ((8 + header.size()) % 256 != 0) header.push_back(' ');  // the tensors start on a 256-byte boundary of the file
    std::FILE* f = std::fopen(path.c_str(), "wb");
    if (f == nullptr) throw std::runtime_error(path + ": cannot create: " + std::strerror(errno));
    bool ok = true;
    unsigned char length[8];
    for (int i = 0; i < 8; ++i) length[i] = static_cast<unsigned char>((static_cast<std::uint64_t>(header.size()) >> (8 * i)) & 0xFF);
    ok = ok && std::fwrite(length, 1, 8, f) == 8;
    ok = ok && std::fwrite(header.data(), 1, header.size(), f) == header.size();
    for (const TensorToWrite& t : tensors) {
        std::uint64_t elements = 1;
        for (const std::uint64_t d : t.shape) elements *= d;
        const std::uint64_t bytes = elements * bytes_of(t.type);
        if (bytes != 0) ok = ok && std::fwrite(t.data, 1, bytes, f) == bytes;
    }
    ok = (std::fclose(f) == 0) && ok;
    if (!ok) throw std::runtime_error(path + ": write failed");
}

}  // namespace sepal::b200
