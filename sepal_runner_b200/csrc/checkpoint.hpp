// Checkpoint files as the weight placement reads them: the safetensors format (an 8-byte little-endian header length, a JSON header
// naming each tensor's "dtype", "shape" and "data_offsets" counted from the end of the header, then the tensors' bytes), mapped
// read-only and checked once, so that every view handed out lies inside the file, has the size its shape and type imply, is aligned
// for its type and overlaps no other tensor. The counterpart of the reference's reader (runner/include/sepal/safetensors.hpp:1-154,
// runner/src/io/safetensors.cpp) and of its checkpoint directories and name prefixes (runner/include/sepal/loader.hpp:5-8).
#pragma once

#include <cstddef>
#include <cstdint>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <string_view>
#include <vector>

namespace sepal::b200 {

enum class ElementType : int { F32 = 0, F16 = 1, BF16 = 2, I8 = 3, U8 = 4, I32 = 5, I64 = 6, F64 = 7, Bool = 8, I16 = 9, U16 = 10, U32 = 11, U64 = 12 };
std::size_t bytes_of(ElementType type);
const char* name_of(ElementType type);

/// A malformed file; the message names the file and, where there is one, the tensor.
class CheckpointError : public std::runtime_error {
public:
    using std::runtime_error::runtime_error;
};

struct TensorView {
    std::string name;
    ElementType type = ElementType::F32;
    std::vector<std::uint64_t> shape;
    const unsigned char* data = nullptr;  // valid while the file object lives
    std::uint64_t bytes = 0;
    std::uint64_t elements() const;
};

/// One parsed file: a read-only mapping, or bytes the caller keeps alive.
class TensorFile {
public:
    static std::shared_ptr<const TensorFile> open(const std::string& path);
    static std::shared_ptr<const TensorFile> from_memory(const unsigned char* bytes, std::size_t size, std::string origin);
    ~TensorFile();
    TensorFile(const TensorFile&) = delete;
    TensorFile& operator=(const TensorFile&) = delete;

    const std::vector<TensorView>& tensors() const { return tensors_; }  // in file order
    const TensorView* find(std::string_view name) const;
    const std::map<std::string, std::string, std::less<>>& metadata() const { return metadata_; }
    const std::string& origin() const { return origin_; }

private:
    TensorFile() = default;
    void parse(const unsigned char* bytes, std::size_t size);
    void* mapping_ = nullptr;
    std::size_t mapped_bytes_ = 0;
    std::string origin_;
    std::vector<TensorView> tensors_;
    std::map<std::string, std::size_t, std::less<>> index_;
    std::map<std::string, std::string, std::less<>> metadata_;
};

/// All tensors of a checkpoint: one file, or a directory holding `model.safetensors` or the shards `model-0000i-of-0000N.safetensors`
/// (all N must be there). The text model's tensors may sit under `model.language_model.`, `language_model.`, `model.` or no prefix: the
/// prefix is found (by `embed_tokens.weight`) and dropped, nothing else is renamed. Two files holding the same name are refused.
class Checkpoint {
public:
    static std::shared_ptr<const Checkpoint> open(const std::string& path);
    static std::shared_ptr<const Checkpoint> from_files(std::vector<std::shared_ptr<const TensorFile>> files);

    const TensorView* find(std::string_view engine_name) const;
    const TensorView& at(std::string_view engine_name) const;  // throws std::out_of_range naming the tensor
    std::vector<std::string> names() const;                    // engine names, sorted
    const std::string& prefix() const { return prefix_; }
    const std::vector<std::shared_ptr<const TensorFile>>& files() const { return files_; }
    /// The value of a metadata key of the first file that has it, or an empty string.
    std::string metadata(std::string_view key) const;

private:
    std::vector<std::shared_ptr<const TensorFile>> files_;
    std::map<std::string, const TensorView*, std::less<>> by_name_;  // full names
    std::string prefix_;
};

/// Writes a file in the same format. Tensors start on 256-byte boundaries of the file (the header is padded with spaces), so that a
/// mapped tensor can be copied to the device, or read by a bulk copy engine, without realignment.
struct TensorToWrite {
    std::string name;
    ElementType type;
    std::vector<std::uint64_t> shape;
    const void* data;  // host
};
void write_tensor_file(const std::string& path, const std::vector<TensorToWrite>& tensors, const std::map<std::string, std::string>& metadata);

}  // namespace sepal::b200
