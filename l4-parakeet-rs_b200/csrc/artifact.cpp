// Reader for the reference's ahead-of-time weight artifact (".pkl4") and the layout packers
// that produce its tensors.  Host code only; nothing here touches a GPU.
//
// File layout (src/artifact.rs:11-16, :98-156, :345-411):
//   bytes 0..8    magic "PKL4AOT\0"
//   bytes 8..12   schema version, u32 little endian (2)
//   bytes 12..16  flags, u32 (0)
//   bytes 16..24  header length in bytes, u64 (1 .. 128 MiB)
//   bytes 24..    JSON header (AotHeader, src/artifact.rs:47-60)
//   payload       starts at align_up(24 + header length, 4096); tensor offsets are relative to
//                 it, 256-byte aligned, in increasing order; the last tensor ends the file.
// Tensor storages (src/artifact.rs:18-34, :687-724): plain fp16 / fp32 (physical shape =
// logical shape), "sm89_fp16_linear" = fp16 [out ^128, in ^128] row-major zero padded,
// "sm89_fp32_bias" = fp32 [out ^128] zero padded.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "../../include/pk100.h"

namespace {

constexpr unsigned char kMagic[8] = {'P', 'K', 'L', '4', 'A', 'O', 'T', 0};
constexpr uint32_t kSchemaVersion = 2;
constexpr uint64_t kPrefixBytes = 24;
constexpr uint64_t kHeaderAlignment = 4096;
constexpr uint64_t kTensorAlignment = 256;
constexpr uint64_t kMaxHeaderBytes = 128ull * 1024 * 1024;

struct FormatError {
    int code;
    std::string message;
};
[[noreturn]] void invalid(const std::string& message) { throw FormatError{PK100_ERR_FORMAT, message}; }

bool align_up_checked(uint64_t value, uint64_t alignment, uint64_t* out) {
    if (alignment == 0 || value > UINT64_MAX - (alignment - 1)) return false;
    *out = (value + alignment - 1) / alignment * alignment;
    return true;
}

// ------------------------------------------------------------------ JSON
// A small document model: enough for the header (objects, arrays, strings, unsigned
// integers; other numbers are kept as doubles, literals as their kind).
struct Json {
    enum Kind { Null, Bool, Unsigned, Number, String, Array, Object } kind = Null;
    bool boolean = false;
    uint64_t integer = 0;
    double number = 0.0;
    std::string text;
    std::vector<Json> items;
    std::vector<std::pair<std::string, Json>> members;

    const Json* get(const char* key) const {
        if (kind != Object) return nullptr;
        for (const auto& m : members)
            if (m.first == key) return &m.second;
        return nullptr;
    }
    // How often `key` occurs: the header and the tensor records are serde-derived structs in the
    // reference (src/artifact.rs:30-60), which refuse a field given twice ("duplicate field")
    // while repeated unknown keys are ignored like any unknown key.
    int count(const char* key) const {
        int n = 0;
        for (const auto& m : members) n += m.first == key ? 1 : 0;
        return n;
    }
};

void reject_duplicate_fields(const Json& object, std::initializer_list<const char*> fields) {
    for (const char* key : fields)
        if (object.count(key) > 1) invalid(std::string("header: duplicate field `") + key + "`");
}

class JsonParser {
public:
    JsonParser(const char* data, size_t size) : p_(data), end_(data + size) {}
    Json parse_document() {
        Json v = parse_value(0);
        skip_space();
        if (p_ != end_) invalid("header: trailing bytes after the JSON document");
        return v;
    }

private:
    const char* p_;
    const char* end_;

    void skip_space() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\t' || *p_ == '\n' || *p_ == '\r')) ++p_;
    }
    [[noreturn]] void fail(const char* what) {
        invalid(std::string("header: ") + what);
    }
    bool consume(const char* literal) {
        const size_t n = std::strlen(literal);
        if (static_cast<size_t>(end_ - p_) < n || std::memcmp(p_, literal, n) != 0) return false;
        p_ += n;
        return true;
    }
    static void append_utf8(std::string& out, uint32_t cp) {
        if (cp < 0x80) {
            out.push_back(static_cast<char>(cp));
        } else if (cp < 0x800) {
            out.push_back(static_cast<char>(0xC0 | (cp >> 6)));
            out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
        } else if (cp < 0x10000) {
            out.push_back(static_cast<char>(0xE0 | (cp >> 12)));
            out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
            out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
        } else {
            out.push_back(static_cast<char>(0xF0 | (cp >> 18)));
            out.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
            out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
            out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
        }
    }
    uint32_t hex4() {
        if (end_ - p_ < 4) fail("truncated \\u escape");
        uint32_t v = 0;
        for (int i = 0; i < 4; ++i) {
            const char c = *p_++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= static_cast<uint32_t>(c - '0');
            else if (c >= 'a' && c <= 'f') v |= static_cast<uint32_t>(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= static_cast<uint32_t>(c - 'A' + 10);
            else fail("bad \\u escape");
        }
        return v;
    }
    std::string parse_string() {
        if (p_ >= end_ || *p_ != '"') fail("expected a string");
        ++p_;
        std::string out;
        while (true) {
            if (p_ >= end_) fail("unterminated string");
            const unsigned char c = static_cast<unsigned char>(*p_++);
            if (c == '"') return out;
            if (c < 0x20) fail("control character inside a string");
            if (c != '\\') {
                out.push_back(static_cast<char>(c));
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
                uint32_t cp = hex4();
                if (cp >= 0xD800 && cp <= 0xDBFF) {           // surrogate pair
                    if (!consume("\\u")) fail("lone high surrogate");
                    const uint32_t low = hex4();
                    if (low < 0xDC00 || low > 0xDFFF) fail("bad low surrogate");
                    cp = 0x10000 + ((cp - 0xD800) << 10) + (low - 0xDC00);
                } else if (cp >= 0xDC00 && cp <= 0xDFFF) {
                    fail("lone low surrogate");
                }
                append_utf8(out, cp);
                break;
            }
            default: fail("unknown escape");
            }
        }
    }
    Json parse_number() {
        const char* start = p_;
        bool plain = true;                     // digits only -> unsigned integer
        if (p_ < end_ && *p_ == '-') { plain = false; ++p_; }
        if (p_ >= end_ || *p_ < '0' || *p_ > '9') fail("bad number");
        while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        if (p_ < end_ && *p_ == '.') {
            plain = false;
            ++p_;
            if (p_ >= end_ || *p_ < '0' || *p_ > '9') fail("bad fraction");
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        if (p_ < end_ && (*p_ == 'e' || *p_ == 'E')) {
            plain = false;
            ++p_;
            if (p_ < end_ && (*p_ == '+' || *p_ == '-')) ++p_;
            if (p_ >= end_ || *p_ < '0' || *p_ > '9') fail("bad exponent");
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        Json v;
        const std::string token(start, p_);
        if (plain) {
            uint64_t acc = 0;
            for (const char c : token) {
                const uint64_t digit = static_cast<uint64_t>(c - '0');
                if (acc > (UINT64_MAX - digit) / 10) fail("integer does not fit 64 bits");
                acc = acc * 10 + digit;
            }
            v.kind = Json::Unsigned;
            v.integer = acc;
        } else {
            v.kind = Json::Number;
            v.number = std::strtod(token.c_str(), nullptr);
        }
        return v;
    }
    Json parse_value(int depth) {
        if (depth > 32) fail("nesting too deep");
        skip_space();
        if (p_ >= end_) fail("unexpected end of header");
        Json v;
        const char c = *p_;
        if (c == '{') {
            ++p_;
            v.kind = Json::Object;
            skip_space();
            if (p_ < end_ && *p_ == '}') { ++p_; return v; }
            while (true) {
                skip_space();
                std::string key = parse_string();
                skip_space();
                if (p_ >= end_ || *p_ != ':') fail("expected ':'");
                ++p_;
                v.members.emplace_back(std::move(key), parse_value(depth + 1));
                skip_space();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == '}') { ++p_; return v; }
                fail("expected ',' or '}'");
            }
        }
        if (c == '[') {
            ++p_;
            v.kind = Json::Array;
            skip_space();
            if (p_ < end_ && *p_ == ']') { ++p_; return v; }
            while (true) {
                v.items.push_back(parse_value(depth + 1));
                skip_space();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == ']') { ++p_; return v; }
                fail("expected ',' or ']'");
            }
        }
        if (c == '"') {
            v.kind = Json::String;
            v.text = parse_string();
            return v;
        }
        if (consume("true")) { v.kind = Json::Bool; v.boolean = true; return v; }
        if (consume("false")) { v.kind = Json::Bool; return v; }
        if (consume("null")) return v;
        return parse_number();
    }
};

// ------------------------------------------------------------------ header model
struct Tensor {
    std::string name;
    int storage = 0;
    std::vector<uint64_t> logical, physical;
    uint64_t offset = 0, bytes = 0;
};

struct Profile {
    const char* key;          // serde name
    const char* repository;
    const char* revision;
    uint64_t blank_token_id;  // = vocabulary entries in the header
};
// src/config.rs:5-55
constexpr Profile kProfiles[] = {
    {"v2_english", "nvidia/parakeet-tdt-0.6b-v2", "ae9ad07059c7c739ffaf932226a8fe64ae2620b0", 1024},
    {"v3_multilingual", "nvidia/parakeet-tdt-0.6b-v3", "541d1f99c6b0c3cd0b11a95167540bb8edefd82b", 8192},
};

const std::string& need_string(const Json& header, const char* key) {
    const Json* v = header.get(key);
    if (v == nullptr || v->kind != Json::String) invalid(std::string("header: missing string field ") + key);
    return v->text;
}
uint64_t need_unsigned(const Json& object, const char* key, const char* where) {
    const Json* v = object.get(key);
    if (v == nullptr || v->kind != Json::Unsigned)
        invalid(std::string(where) + ": missing unsigned integer field " + key);
    return v->integer;
}
std::vector<uint64_t> need_shape(const Json& object, const char* key, const std::string& name) {
    const Json* v = object.get(key);
    if (v == nullptr || v->kind != Json::Array) invalid(name + ": missing array field " + key);
    std::vector<uint64_t> shape;
    for (const Json& d : v->items) {
        if (d.kind != Json::Unsigned) invalid(name + ": " + key + " holds a non-integer");
        shape.push_back(d.integer);
    }
    if (shape.size() > 4) invalid(name + ": rank above 4");
    return shape;
}
int storage_from(const std::string& text, const std::string& name) {
    if (text == "fp16") return PK100_STORAGE_FP16;
    if (text == "fp32") return PK100_STORAGE_FP32;
    if (text == "sm89_fp16_linear") return PK100_STORAGE_FP16_LINEAR;
    if (text == "sm89_fp32_bias") return PK100_STORAGE_FP32_BIAS;
    invalid(name + ": unknown storage " + text);
}
uint64_t element_bytes(int storage) {
    return (storage == PK100_STORAGE_FP16 || storage == PK100_STORAGE_FP16_LINEAR) ? 2 : 4;
}
uint64_t checked_elements(const std::vector<uint64_t>& shape, const std::string& name) {
    uint64_t n = 1;
    for (const uint64_t d : shape) {
        if (d != 0 && n > UINT64_MAX / d) invalid(name + ": element count overflow");
        n *= d;
    }
    return n;
}
std::string shape_text(const std::vector<uint64_t>& shape) {
    std::string s = "[";
    for (size_t i = 0; i < shape.size(); ++i) s += (i ? ", " : "") + std::to_string(shape[i]);
    return s + "]";
}

// src/artifact.rs:687-724
void validate_tensor_layout(const Tensor& t) {
    auto aligned = [&](uint64_t d) {
        uint64_t out = 0;
        if (!align_up_checked(d, 128, &out)) invalid(t.name + ": alignment overflow");
        return out;
    };
    switch (t.storage) {
    case PK100_STORAGE_FP16:
    case PK100_STORAGE_FP32:
        if (t.physical != t.logical)
            invalid(t.name + ": plain storage cannot change logical shape " + shape_text(t.logical) + " to " +
                    shape_text(t.physical));
        break;
    case PK100_STORAGE_FP16_LINEAR:
        if (!(t.logical.size() == 2 && t.logical[0] > 0 && t.logical[1] > 0 && t.physical.size() == 2 &&
              t.physical[0] == aligned(t.logical[0]) && t.physical[1] == aligned(t.logical[1])))
            invalid(t.name + ": invalid sm_89 FP16 linear shapes " + shape_text(t.logical) + " -> " +
                    shape_text(t.physical));
        break;
    default:
        if (!(t.logical.size() == 1 && t.logical[0] > 0 && t.physical.size() == 1 &&
              t.physical[0] == aligned(t.logical[0])))
            invalid(t.name + ": invalid sm_89 FP32 bias shapes " + shape_text(t.logical) + " -> " +
                    shape_text(t.physical));
    }
}

}  // namespace

struct pk100_artifact {
    int fd = -1;
    const unsigned char* map = nullptr;
    uint64_t file_bytes = 0, data_start = 0;
    std::map<std::string, std::string> fields;
    std::vector<std::string> vocabulary;
    std::vector<Tensor> tensors;
    std::map<std::string, int> index;

    ~pk100_artifact() {
        if (map != nullptr) munmap(const_cast<unsigned char*>(map), file_bytes);
        if (fd >= 0) close(fd);
    }
};

namespace {

uint32_t le32(const unsigned char* p) { return p[0] | (p[1] << 8) | (p[2] << 16) | (static_cast<uint32_t>(p[3]) << 24); }
uint64_t le64(const unsigned char* p) { return le32(p) | (static_cast<uint64_t>(le32(p + 4)) << 32); }

// src/artifact.rs:99-156 (open) and :514-593 (validate_header)
void load(pk100_artifact& a, const char* path) {
    a.fd = open(path, O_RDONLY);
    if (a.fd < 0) throw FormatError{PK100_ERR_IO, std::string("failed to access ") + path + ": " + std::strerror(errno)};
    struct stat st{};
    if (fstat(a.fd, &st) != 0)
        throw FormatError{PK100_ERR_IO, std::string("failed to access ") + path + ": " + std::strerror(errno)};
    a.file_bytes = static_cast<uint64_t>(st.st_size);
    if (a.file_bytes < kPrefixBytes)
        invalid("file has " + std::to_string(a.file_bytes) + " bytes; prefix requires " + std::to_string(kPrefixBytes));
    void* m = mmap(nullptr, a.file_bytes, PROT_READ, MAP_PRIVATE, a.fd, 0);
    if (m == MAP_FAILED)
        throw FormatError{PK100_ERR_IO, std::string("failed to map ") + path + ": " + std::strerror(errno)};
    a.map = static_cast<const unsigned char*>(m);

    if (std::memcmp(a.map, kMagic, 8) != 0) invalid("bad magic");
    const uint32_t version = le32(a.map + 8), flags = le32(a.map + 12);
    const uint64_t header_bytes = le64(a.map + 16);
    if (version != kSchemaVersion)
        invalid("expected schema version " + std::to_string(kSchemaVersion) + ", got " + std::to_string(version));
    if (flags != 0) invalid("unsupported prefix flags " + std::to_string(flags));
    if (header_bytes == 0 || header_bytes > kMaxHeaderBytes)
        invalid("header length " + std::to_string(header_bytes) + " is outside 1..=" + std::to_string(kMaxHeaderBytes));
    uint64_t data_start = 0;
    if (!align_up_checked(kPrefixBytes + header_bytes, kHeaderAlignment, &data_start)) invalid("header offset overflow");
    if (data_start > a.file_bytes)
        invalid("aligned header ends at " + std::to_string(data_start) + ", beyond file length " +
                std::to_string(a.file_bytes));
    a.data_start = data_start;
    const uint64_t payload_bytes = a.file_bytes - data_start;

    const Json header = JsonParser(reinterpret_cast<const char*>(a.map + kPrefixBytes), header_bytes).parse_document();
    if (header.kind != Json::Object) invalid("header: not a JSON object");
    reject_duplicate_fields(header, {"schema_version", "target", "profile", "source_repository", "source_revision",
                                     "source_payload_bytes", "precision_plan", "tensor_alignment", "payload_bytes",
                                     "vocabulary", "tensors"});

    if (need_unsigned(header, "schema_version", "header") != kSchemaVersion)
        invalid("header schema is " + std::to_string(need_unsigned(header, "schema_version", "header")) +
                ", expected " + std::to_string(kSchemaVersion));
    for (const char* key : {"target", "profile", "source_repository", "source_revision", "precision_plan"})
        a.fields[key] = need_string(header, key);
    need_unsigned(header, "source_payload_bytes", "header");
    // "sm_89" is what the reference writes; the layouts are the ones these kernels read, so the
    // same file is accepted, as is one re-tagged for this target
    if (a.fields["target"] != "sm_89" && a.fields["target"] != "sm_100a")
        invalid("target is \"" + a.fields["target"] + "\", expected sm_89");
    const Profile* profile = nullptr;
    for (const Profile& p : kProfiles)
        if (a.fields["profile"] == p.key) profile = &p;
    if (profile == nullptr) invalid("header: unknown profile " + a.fields["profile"]);
    if (a.fields["source_repository"] != profile->repository || a.fields["source_revision"] != profile->revision)
        invalid("profile does not match source repository and revision");
    if (need_unsigned(header, "tensor_alignment", "header") != kTensorAlignment)
        invalid("tensor alignment is " + std::to_string(need_unsigned(header, "tensor_alignment", "header")) +
                ", expected " + std::to_string(kTensorAlignment));
    if (need_unsigned(header, "payload_bytes", "header") != payload_bytes)
        invalid("header declares " + std::to_string(need_unsigned(header, "payload_bytes", "header")) +
                " payload bytes, file contains " + std::to_string(payload_bytes));

    const Json* vocabulary = header.get("vocabulary");
    if (vocabulary == nullptr || vocabulary->kind != Json::Array) invalid("header: missing array field vocabulary");
    if (vocabulary->items.size() != profile->blank_token_id)
        invalid(a.fields["profile"] + " requires " + std::to_string(profile->blank_token_id) +
                " vocabulary entries before the blank token, got " + std::to_string(vocabulary->items.size()));
    for (size_t i = 0; i < vocabulary->items.size(); ++i) {
        const Json& piece = vocabulary->items[i];
        if (piece.kind != Json::String) invalid("vocabulary entry " + std::to_string(i) + " is not a string");
        if (piece.text.empty() || piece.text.find_first_of("\n\r\t") != std::string::npos)
            invalid("vocabulary entry " + std::to_string(i) + " is empty or contains control separators");
        a.vocabulary.push_back(piece.text);
    }

    const Json* tensors = header.get("tensors");
    if (tensors == nullptr || tensors->kind != Json::Array) invalid("header: missing array field tensors");
    uint64_t cursor = 0;
    for (const Json& record : tensors->items) {
        if (record.kind != Json::Object) invalid("header: tensor record is not an object");
        reject_duplicate_fields(record, {"name", "storage", "logical_shape", "physical_shape", "offset", "bytes"});
        Tensor t;
        const Json* name = record.get("name");
        if (name == nullptr || name->kind != Json::String) invalid("header: tensor record without a name");
        t.name = name->text;
        if (t.name.empty() || a.index.count(t.name) != 0) invalid("empty or duplicate tensor name \"" + t.name + "\"");
        const Json* storage = record.get("storage");
        if (storage == nullptr || storage->kind != Json::String) invalid(t.name + ": missing storage");
        t.storage = storage_from(storage->text, t.name);
        t.logical = need_shape(record, "logical_shape", t.name);
        t.physical = need_shape(record, "physical_shape", t.name);
        t.offset = need_unsigned(record, "offset", t.name.c_str());
        t.bytes = need_unsigned(record, "bytes", t.name.c_str());
        if (t.offset % kTensorAlignment != 0 || t.offset < cursor)
            invalid(t.name + ": invalid aligned offset " + std::to_string(t.offset) + " after " + std::to_string(cursor));
        validate_tensor_layout(t);
        const uint64_t elements = checked_elements(t.physical, t.name);
        if (elements > UINT64_MAX / element_bytes(t.storage)) invalid(t.name + ": byte count overflow");
        const uint64_t expected = elements * element_bytes(t.storage);
        if (t.bytes != expected)
            invalid(t.name + ": physical shape and storage require " + std::to_string(expected) +
                    " bytes, header declares " + std::to_string(t.bytes));
        if (t.offset > UINT64_MAX - t.bytes) invalid(t.name + ": range overflow");
        cursor = t.offset + t.bytes;
        if (cursor > payload_bytes)
            invalid(t.name + ": range ends at " + std::to_string(cursor) + ", beyond " + std::to_string(payload_bytes) +
                    "-byte payload");
        a.index[t.name] = static_cast<int>(a.tensors.size());
        a.tensors.push_back(std::move(t));
    }
    if (cursor != payload_bytes)
        invalid("last tensor ends at " + std::to_string(cursor) + ", payload ends at " + std::to_string(payload_bytes));
}

// IEEE binary32 -> binary16, round to nearest even (what half::f16::from_f32 does).
uint16_t f32_to_f16_rne(float value) {
    uint32_t x;
    std::memcpy(&x, &value, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t mag = x & 0x7FFFFFFFu;
    if (mag >= 0x7F800000u) return static_cast<uint16_t>(sign | (mag > 0x7F800000u ? 0x7E00u : 0x7C00u));
    if (mag >= 0x477FF000u) return static_cast<uint16_t>(sign | 0x7C00u);      // rounds to infinity
    if (mag >= 0x38800000u) {                                                    // normal half
        const uint32_t rebased = mag - 0x38000000u;                              // exponent 127 -> 15
        const uint32_t rounded = rebased + 0x0FFFu + ((rebased >> 13) & 1u);
        return static_cast<uint16_t>(sign | (rounded >> 13));
    }
    if (mag < 0x33000000u) return static_cast<uint16_t>(sign);                   // below half of the smallest subnormal
    // subnormal half: value = mantissa24 * 2^(e - 150); target unit 2^-24
    const uint32_t e = mag >> 23;
    const uint32_t mantissa = (mag & 0x007FFFFFu) | 0x00800000u;
    const uint32_t shift = 126 - e;                                              // 14 .. 24
    const uint32_t kept = mantissa >> shift;
    const uint32_t rest = mantissa & ((1u << shift) - 1u);
    const uint32_t half_way = 1u << (shift - 1);
    const uint32_t up = (rest > half_way || (rest == half_way && (kept & 1u))) ? 1u : 0u;
    return static_cast<uint16_t>(sign | (kept + up));
}

void copy_error(const std::string& message, char* error, int error_len) {
    if (error == nullptr || error_len <= 0) return;
    std::snprintf(error, static_cast<size_t>(error_len), "%s", message.c_str());
}

}  // namespace

extern "C" int pk100_artifact_open(const char* path, pk100_artifact** out, char* error, int error_len) {
    if (out == nullptr || path == nullptr) return PK100_ERR_NULL;
    *out = nullptr;
    std::unique_ptr<pk100_artifact> a(new pk100_artifact());
    try {
        load(*a, path);
    } catch (const FormatError& e) {
        copy_error(e.message, error, error_len);
        return e.code;
    } catch (const std::exception& e) {
        copy_error(e.what(), error, error_len);
        return PK100_ERR_FORMAT;
    }
    *out = a.release();
    return PK100_OK;
}

extern "C" void pk100_artifact_close(pk100_artifact* artifact) { delete artifact; }

extern "C" int pk100_artifact_tensor_count(const pk100_artifact* a) {
    return a == nullptr ? 0 : static_cast<int>(a->tensors.size());
}

extern "C" int pk100_artifact_tensor_at(const pk100_artifact* a, int index, pk100_artifact_tensor* out) {
    if (a == nullptr || out == nullptr) return PK100_ERR_NULL;
    if (index < 0 || index >= static_cast<int>(a->tensors.size())) return PK100_ERR_SHAPE;
    const Tensor& t = a->tensors[static_cast<size_t>(index)];
    std::memset(out, 0, sizeof(*out));
    out->name = t.name.c_str();
    out->storage = t.storage;
    out->logical_rank = static_cast<int>(t.logical.size());
    out->physical_rank = static_cast<int>(t.physical.size());
    for (size_t i = 0; i < t.logical.size(); ++i) out->logical_shape[i] = static_cast<long long>(t.logical[i]);
    for (size_t i = 0; i < t.physical.size(); ++i) out->physical_shape[i] = static_cast<long long>(t.physical[i]);
    out->offset = t.offset;
    out->bytes = t.bytes;
    out->data = a->map + a->data_start + t.offset;
    return PK100_OK;
}

extern "C" int pk100_artifact_find(const pk100_artifact* a, const char* name) {
    if (a == nullptr || name == nullptr) return -1;
    const auto it = a->index.find(name);
    return it == a->index.end() ? -1 : it->second;
}

extern "C" int pk100_artifact_vocabulary_size(const pk100_artifact* a) {
    return a == nullptr ? 0 : static_cast<int>(a->vocabulary.size());
}

extern "C" const char* pk100_artifact_vocabulary_at(const pk100_artifact* a, int index) {
    if (a == nullptr || index < 0 || index >= static_cast<int>(a->vocabulary.size())) return nullptr;
    return a->vocabulary[static_cast<size_t>(index)].c_str();
}

extern "C" const char* pk100_artifact_field(const pk100_artifact* a, const char* key) {
    if (a == nullptr || key == nullptr) return nullptr;
    const auto it = a->fields.find(key);
    return it == a->fields.end() ? nullptr : it->second.c_str();
}

// src/artifact.rs:158-187: plain FP32 tensors only, every value finite.
extern "C" int pk100_artifact_read_f32(const pk100_artifact* a, const char* name, float* out, long long capacity) {
    if (a == nullptr || name == nullptr || out == nullptr) return PK100_ERR_NULL;
    const int index = pk100_artifact_find(a, name);
    if (index < 0) return PK100_ERR_FORMAT;
    const Tensor& t = a->tensors[static_cast<size_t>(index)];
    if (t.storage != PK100_STORAGE_FP32 || t.logical != t.physical) return PK100_ERR_FORMAT;
    const long long elements = static_cast<long long>(t.bytes / 4);
    if (capacity < elements) return PK100_ERR_SHAPE;
    std::memcpy(out, a->map + a->data_start + t.offset, t.bytes);
    for (long long i = 0; i < elements; ++i)
        if (!std::isfinite(out[i])) return PK100_ERR_FORMAT;
    return PK100_OK;
}

// ------------------------------------------------------------------ layout packers
// src/artifact.rs:413-428
extern "C" int pk100_encode_fp16(const float* source, long long elements, uint16_t* out) {
    if (source == nullptr || out == nullptr) return PK100_ERR_NULL;
    if (elements < 0) return PK100_ERR_SHAPE;
    for (long long i = 0; i < elements; ++i) {
        if (!std::isfinite(source[i])) return PK100_ERR_FORMAT;
        out[i] = f32_to_f16_rne(source[i]);
    }
    return PK100_OK;
}

// src/artifact.rs:430-467: [logical_out, logical_in] fp32 -> [padded_out, padded_in] fp16, zero padded.
extern "C" int pk100_encode_fp16_linear(const float* source, long long logical_out, long long logical_in,
                                        long long padded_out, long long padded_in, uint16_t* out) {
    if (source == nullptr || out == nullptr) return PK100_ERR_NULL;
    if (logical_out < 0 || logical_in < 0 || padded_out < logical_out || padded_in < logical_in) return PK100_ERR_SHAPE;
    std::memset(out, 0, static_cast<size_t>(padded_out) * static_cast<size_t>(padded_in) * 2);
    for (long long row = 0; row < logical_out; ++row)
        for (long long column = 0; column < logical_in; ++column) {
            const float v = source[row * logical_in + column];
            if (!std::isfinite(v)) return PK100_ERR_FORMAT;
            out[row * padded_in + column] = f32_to_f16_rne(v);
        }
    return PK100_OK;
}

// src/artifact.rs:469-484
extern "C" int pk100_encode_fp32_bias(const float* source, long long logical, long long padded, float* out) {
    if (source == nullptr || out == nullptr) return PK100_ERR_NULL;
    if (logical < 0 || padded < logical) return PK100_ERR_SHAPE;
    for (long long i = 0; i < logical; ++i)
        if (!std::isfinite(source[i])) return PK100_ERR_FORMAT;
    std::memset(out, 0, static_cast<size_t>(padded) * 4);
    std::memcpy(out, source, static_cast<size_t>(logical) * 4);
    return PK100_OK;
}

// src/artifact.rs:734-739: returns 0 and sets *overflow when value + alignment - 1 does not fit.
extern "C" unsigned long long pk100_align_up(unsigned long long value, unsigned long long alignment, int* overflow) {
    uint64_t out = 0;
    const bool ok = align_up_checked(value, alignment, &out);
    if (overflow != nullptr) *overflow = ok ? 0 : 1;
    return ok ? out : 0;
}

// ---------------------------------------------------------------------------
// Packed-layout size contract (src/packing.rs:5-130, src/exl3.rs:14-75): byte counts and padded
// shapes of the five candidate weight formats.  Pure integer arithmetic with overflow checks.
namespace {
constexpr uint64_t kTileAlignment = 128;      // TILE_ALIGNMENT, HADAMARD_BLOCK, OUTPUT_ALIGNMENT
constexpr uint64_t kTrellisTile = 16;
constexpr uint64_t kQ4kBlockElements = 256, kQ4kBlockBytes = 144;

bool mul3(uint64_t a, uint64_t b, uint64_t c, uint64_t* out) {
    uint64_t ab = 0;
    if (__builtin_mul_overflow(a, b, &ab)) return false;
    return !__builtin_mul_overflow(ab, c, out);
}
}  // namespace

extern "C" int pk100_exl3_layout(long long logical_in, long long logical_out, int qbits, pk100_exl3_layout_t* out) {
    if (out == nullptr) return PK100_ERR_NULL;
    if (logical_in <= 0 || logical_out <= 0) return PK100_ERR_SHAPE;          // Exl3LayoutError::Empty
    if (qbits < 1 || qbits > 8) return PK100_ERR_UNSUPPORTED;                  // InvalidBitRate
    uint64_t pi = 0, po = 0, bits = 0;
    if (!align_up_checked(static_cast<uint64_t>(logical_in), kTileAlignment, &pi) ||
        !align_up_checked(static_cast<uint64_t>(logical_out), kTileAlignment, &po) ||
        !mul3(pi, po, static_cast<uint64_t>(qbits), &bits))
        return PK100_ERR_LIMIT;
    out->padded_in = static_cast<long long>(pi);
    out->padded_out = static_cast<long long>(po);
    out->trellis_shape[0] = static_cast<long long>(pi / kTrellisTile);
    out->trellis_shape[1] = static_cast<long long>(po / kTrellisTile);
    out->trellis_shape[2] = static_cast<long long>(kTrellisTile * static_cast<uint64_t>(qbits));
    out->trellis_bytes = bits / 8;
    out->scale_bytes = 2 * (pi + po);
    return PK100_OK;
}

extern "C" int pk100_estimate_linear(int format, long long logical_in, long long logical_out, int exl3_bits,
                                     pk100_linear_layout* out) {
    if (out == nullptr) return PK100_ERR_NULL;
    if (logical_in <= 0 || logical_out <= 0) return PK100_ERR_SHAPE;          // PackingError::Empty
    const uint64_t in = static_cast<uint64_t>(logical_in), outw = static_cast<uint64_t>(logical_out);
    uint64_t pi = 0, po = 0, payload = 0, meta = 0;
    out->logical_in = logical_in;
    out->logical_out = logical_out;
    out->available = 1;
    switch (format) {
    case PK100_FORMAT_FP16:
    case PK100_FORMAT_FP8_E4M3:
    case PK100_FORMAT_INT8:
        if (!align_up_checked(in, kTileAlignment, &pi) || !align_up_checked(outw, kTileAlignment, &po)) return PK100_ERR_LIMIT;
        if (!mul3(pi, po, format == PK100_FORMAT_FP16 ? 2 : 1, &payload)) return PK100_ERR_LIMIT;
        if (format != PK100_FORMAT_FP16 && __builtin_mul_overflow(po, uint64_t{4}, &meta)) return PK100_ERR_LIMIT;
        break;
    case PK100_FORMAT_Q4_K:
        pi = in; po = outw;
        if (in % kQ4kBlockElements != 0) {            // Ok(None): the format has no layout for this K
            out->available = 0;
            out->padded_in = out->padded_out = 0;
            out->payload_bytes = out->metadata_bytes = 0;
            return PK100_OK;
        }
        if (!mul3(outw, in / kQ4kBlockElements, kQ4kBlockBytes, &payload)) return PK100_ERR_LIMIT;
        break;
    case PK100_FORMAT_EXL3: {
        pk100_exl3_layout_t lay;
        const int rc = pk100_exl3_layout(logical_in, logical_out, exl3_bits, &lay);
        if (rc != PK100_OK) return rc;
        pi = static_cast<uint64_t>(lay.padded_in); po = static_cast<uint64_t>(lay.padded_out);
        payload = lay.trellis_bytes; meta = lay.scale_bytes;
        break;
    }
    default:
        return PK100_ERR_UNSUPPORTED;
    }
    out->padded_in = static_cast<long long>(pi);
    out->padded_out = static_cast<long long>(po);
    out->payload_bytes = payload;
    out->metadata_bytes = meta;
    return PK100_OK;
}
