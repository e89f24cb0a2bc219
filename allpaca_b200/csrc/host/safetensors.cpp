#include "safetensors.hpp"

#include <cerrno>
#include <cstring>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <unordered_set>

namespace allpaca {
namespace {

// ---- a JSON reader, as much of it as a safetensors header needs (all of the grammar; numbers
// are kept as integers where they are written as such) -----------------------------------------
struct JValue {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool boolean = false;
    bool is_integer = false;
    int64_t integer = 0;
    double number = 0.0;
    std::string string;
    std::vector<JValue> array;
    std::vector<std::pair<std::string, JValue>> object;   // in the order written
};

class JsonReader {
public:
    JsonReader(const char* p, size_t n) : begin_(p), p_(p), end_(p + n) {}

    bool parse(JValue* out, std::string* error) {
        skip();
        if (!value(out, 0)) { *error = error_ + " at byte " + std::to_string(at_); return false; }
        skip();
        if (p_ != end_) { *error = "text after the value at byte " + std::to_string(p_ - begin_); return false; }
        return true;
    }

private:
    static constexpr int kMaxDepth = 64;
    const char* begin_;
    const char* p_;
    const char* end_;
    std::string error_;
    size_t at_ = 0;

    bool fail(const char* what) {
        error_ = what;
        at_ = (size_t)(p_ - begin_);
        return false;
    }
    char peek() const { return p_ < end_ ? *p_ : '\0'; }
    void advance() { ++p_; }
    void skip() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\t' || *p_ == '\n' || *p_ == '\r')) advance();
    }
    bool literal(const char* word) {
        const size_t n = std::strlen(word);
        if ((size_t)(end_ - p_) < n || std::memcmp(p_, word, n) != 0) return fail("unknown literal");
        p_ += n;
        return true;
    }
    static void put_utf8(std::string* s, uint32_t cp) {
        if (cp < 0x80) s->push_back((char)cp);
        else if (cp < 0x800) { s->push_back((char)(0xC0 | (cp >> 6))); s->push_back((char)(0x80 | (cp & 0x3F))); }
        else if (cp < 0x10000) {
            s->push_back((char)(0xE0 | (cp >> 12)));
            s->push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
            s->push_back((char)(0x80 | (cp & 0x3F)));
        } else {
            s->push_back((char)(0xF0 | (cp >> 18)));
            s->push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
            s->push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
            s->push_back((char)(0x80 | (cp & 0x3F)));
        }
    }
    bool hex4(uint32_t* out) {
        if (end_ - p_ < 4) return fail("short \\u escape");
        uint32_t v = 0;
        for (int i = 0; i < 4; ++i) {
            const char c = p_[i];
            v <<= 4;
            if (c >= '0' && c <= '9') v |= (uint32_t)(c - '0');
            else if (c >= 'a' && c <= 'f') v |= (uint32_t)(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= (uint32_t)(c - 'A' + 10);
            else return fail("bad \\u escape");
        }
        p_ += 4;
        *out = v;
        return true;
    }
    bool string(std::string* out) {
        if (peek() != '"') return fail("a string was expected");
        advance();
        out->clear();
        while (p_ < end_) {
            const unsigned char c = (unsigned char)*p_;
            if (c == '"') { advance(); return true; }
            if (c < 0x20) return fail("control character in a string");
            if (c != '\\') { out->push_back((char)c); advance(); continue; }
            advance();
            if (p_ >= end_) break;
            const char e = *p_;
            advance();
            switch (e) {
                case '"': out->push_back('"'); break;
                case '\\': out->push_back('\\'); break;
                case '/': out->push_back('/'); break;
                case 'b': out->push_back('\b'); break;
                case 'f': out->push_back('\f'); break;
                case 'n': out->push_back('\n'); break;
                case 'r': out->push_back('\r'); break;
                case 't': out->push_back('\t'); break;
                case 'u': {
                    uint32_t cp;
                    if (!hex4(&cp)) return false;
                    if (cp >= 0xD800 && cp < 0xDC00) {                     // a surrogate pair
                        uint32_t lo;
                        if (end_ - p_ < 2 || p_[0] != '\\' || p_[1] != 'u') return fail("lone surrogate");
                        p_ += 2;
                        if (!hex4(&lo)) return false;
                        if (lo < 0xDC00 || lo > 0xDFFF) return fail("lone surrogate");
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    } else if (cp >= 0xDC00 && cp <= 0xDFFF) {
                        return fail("lone surrogate");
                    }
                    put_utf8(out, cp);
                    break;
                }
                default: return fail("unknown escape");
            }
        }
        return fail("unterminated string");
    }
    bool number(JValue* out) {
        const char* s = p_;
        if (peek() == '-') advance();
        if (!(peek() >= '0' && peek() <= '9')) return fail("a digit was expected");
        if (peek() == '0') advance();
        else while (peek() >= '0' && peek() <= '9') advance();
        bool integer = true;
        if (peek() == '.') {
            integer = false;
            advance();
            if (!(peek() >= '0' && peek() <= '9')) return fail("a digit was expected after the point");
            while (peek() >= '0' && peek() <= '9') advance();
        }
        if (peek() == 'e' || peek() == 'E') {
            integer = false;
            advance();
            if (peek() == '+' || peek() == '-') advance();
            if (!(peek() >= '0' && peek() <= '9')) return fail("a digit was expected in the exponent");
            while (peek() >= '0' && peek() <= '9') advance();
        }
        const std::string text(s, (size_t)(p_ - s));
        out->kind = JValue::Number;
        out->number = std::strtod(text.c_str(), nullptr);
        out->is_integer = false;
        if (integer && text.size() <= 19) {          // fits 64 bits for certain up to 18 digits and a sign
            errno = 0;
            const long long v = std::strtoll(text.c_str(), nullptr, 10);
            if (errno == 0) { out->is_integer = true; out->integer = v; }
        }
        return true;
    }
    bool value(JValue* out, int depth) {
        if (depth > kMaxDepth) return fail("nested too deeply");
        skip();
        const char c = peek();
        if (c == '{') {
            advance();
            out->kind = JValue::Object;
            skip();
            if (peek() == '}') { advance(); return true; }
            for (;;) {
                skip();
                std::string key;
                if (!string(&key)) return false;
                skip();
                if (peek() != ':') return fail("a colon was expected");
                advance();
                JValue v;
                if (!value(&v, depth + 1)) return false;
                out->object.emplace_back(std::move(key), std::move(v));
                skip();
                if (peek() == ',') { advance(); continue; }
                if (peek() == '}') { advance(); return true; }
                return fail("a comma or a closing brace was expected");
            }
        }
        if (c == '[') {
            advance();
            out->kind = JValue::Array;
            skip();
            if (peek() == ']') { advance(); return true; }
            for (;;) {
                JValue v;
                if (!value(&v, depth + 1)) return false;
                out->array.push_back(std::move(v));
                skip();
                if (peek() == ',') { advance(); continue; }
                if (peek() == ']') { advance(); return true; }
                return fail("a comma or a closing bracket was expected");
            }
        }
        if (c == '"') { out->kind = JValue::String; return string(&out->string); }
        if (c == 't') { out->kind = JValue::Bool; out->boolean = true; return literal("true"); }
        if (c == 'f') { out->kind = JValue::Bool; out->boolean = false; return literal("false"); }
        if (c == 'n') { out->kind = JValue::Null; return literal("null"); }
        if (c == '-' || (c >= '0' && c <= '9')) return number(out);
        return fail(p_ >= end_ ? "the text ends early" : "a value was expected");
    }
};

bool valid_utf8(const uint8_t* s, size_t n) {
    size_t i = 0;
    while (i < n) {
        const uint8_t c = s[i];
        size_t more;
        uint32_t cp;
        if (c < 0x80) { ++i; continue; }
        else if ((c & 0xE0) == 0xC0) { more = 1; cp = c & 0x1F; }
        else if ((c & 0xF0) == 0xE0) { more = 2; cp = c & 0x0F; }
        else if ((c & 0xF8) == 0xF0) { more = 3; cp = c & 0x07; }
        else return false;
        if (i + more >= n) return false;
        for (size_t k = 1; k <= more; ++k) {
            if ((s[i + k] & 0xC0) != 0x80) return false;
            cp = (cp << 6) | (s[i + k] & 0x3F);
        }
        if ((more == 1 && cp < 0x80) || (more == 2 && cp < 0x800) || (more == 3 && cp < 0x10000)) return false;   // overlong
        if (cp > 0x10FFFF || (cp >= 0xD800 && cp <= 0xDFFF)) return false;
        i += more + 1;
    }
    return true;
}

std::string quoted(const std::string& s) { return "'" + s + "'"; }

std::string shape_text(const std::vector<int64_t>& shape) {
    std::string t = "[";
    for (size_t i = 0; i < shape.size(); ++i) t += (i ? ", " : "") + std::to_string(shape[i]);
    return t + "]";
}

bool non_negative_integer(const JValue& v, int64_t* out) {
    if (v.kind != JValue::Number || !v.is_integer || v.integer < 0) return false;
    *out = v.integer;
    return true;
}

}  // namespace

int SafetensorsFile::element_size(const std::string& dtype) {
    if (dtype == "F64" || dtype == "I64") return 8;
    if (dtype == "F32" || dtype == "I32") return 4;
    if (dtype == "F16" || dtype == "BF16" || dtype == "I16") return 2;
    if (dtype == "I8" || dtype == "U8" || dtype == "BOOL") return 1;
    return 0;
}

SafetensorsFile::~SafetensorsFile() {
    if (map_) munmap(map_, map_len_);
}

SafetensorsFile* SafetensorsFile::open(const std::string& path, std::string* error) {
    const int fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
    if (fd < 0) {
        *error = "cannot open " + path + ": " + std::strerror(errno);
        return nullptr;
    }
    struct stat st;
    if (fstat(fd, &st) != 0 || !S_ISREG(st.st_mode)) {
        *error = "cannot open " + path + ": not a regular file";
        ::close(fd);
        return nullptr;
    }
    const uint64_t size = (uint64_t)st.st_size;
    if (size < 8) {
        *error = path + ": file of " + std::to_string(size) + " bytes is too short for a header length";
        ::close(fd);
        return nullptr;
    }
    void* map = mmap(nullptr, (size_t)size, PROT_READ, MAP_PRIVATE, fd, 0);
    const int map_errno = errno;
    ::close(fd);                                   // the mapping outlives the descriptor
    if (map == MAP_FAILED) {
        *error = "cannot map " + path + ": " + std::strerror(map_errno);
        return nullptr;
    }
    SafetensorsFile* f = new SafetensorsFile();
    f->map_ = (uint8_t*)map;
    f->map_len_ = (size_t)size;
    auto give_up = [&](const std::string& why) -> SafetensorsFile* {
        *error = path + ": " + why;
        delete f;
        return nullptr;
    };
    uint64_t hlen = 0;
    for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | f->map_[i];       // little-endian
    if (hlen == 0 || hlen > kMaxHeaderBytes)
        return give_up("header length " + std::to_string(hlen) + " is outside 1.." + std::to_string(kMaxHeaderBytes));
    if (8 + hlen > size)
        return give_up("header of " + std::to_string(hlen) + " bytes overruns the file of " + std::to_string(size) +
                       " bytes");
    if (!valid_utf8(f->map_ + 8, (size_t)hlen)) return give_up("header is not UTF-8");
    JValue header;
    std::string why;
    JsonReader reader((const char*)f->map_ + 8, (size_t)hlen);
    if (!reader.parse(&header, &why)) return give_up("header is not JSON: " + why);
    if (header.kind != JValue::Object) return give_up("header is not a JSON object");
    f->data_start_ = (int64_t)(8 + hlen);
    f->data_len_ = (int64_t)(size - 8 - hlen);
    std::unordered_set<std::string> seen;
    for (auto& item : header.object) {
        const std::string& name = item.first;
        const JValue& e = item.second;
        // names and metadata leave this library as C strings
        if (name == "__metadata__") {
            if (e.kind == JValue::Object)
                for (auto& kv : e.object) {
                    if (kv.second.kind != JValue::String) continue;
                    if (kv.first.find('\0') != std::string::npos || kv.second.string.find('\0') != std::string::npos)
                        return give_up("metadata holds a NUL character");
                    f->metadata_.emplace_back(kv.first, kv.second.string);
                }
            continue;
        }
        if (name.find('\0') != std::string::npos) return give_up("a tensor's name holds a NUL character");
        if (!seen.insert(name).second) return give_up("tensor " + quoted(name) + " appears twice in the header");
        const JValue *dtype = nullptr, *shape = nullptr, *offsets = nullptr;
        if (e.kind == JValue::Object)
            for (auto& kv : e.object) {
                if (kv.first == "dtype") dtype = &kv.second;
                else if (kv.first == "shape") shape = &kv.second;
                else if (kv.first == "data_offsets") offsets = &kv.second;
            }
        TensorEntry t;
        t.name = name;
        bool fine = dtype && shape && offsets && dtype->kind == JValue::String && shape->kind == JValue::Array &&
                    offsets->kind == JValue::Array && offsets->array.size() == 2 &&
                    non_negative_integer(offsets->array[0], &t.begin) && non_negative_integer(offsets->array[1], &t.end);
        if (fine)
            for (const JValue& d : shape->array) {
                int64_t dim;
                if (!non_negative_integer(d, &dim)) { fine = false; break; }
                t.shape.push_back(dim);
            }
        if (!fine) return give_up("malformed entry for tensor " + quoted(name));
        t.dtype = dtype->string;
        const int esize = element_size(t.dtype);
        if (esize == 0) return give_up("tensor " + quoted(name) + " has unsupported dtype " + quoted(t.dtype));
        if (!(t.begin <= t.end && t.end <= f->data_len_))
            return give_up("tensor " + quoted(name) + " data [" + std::to_string(t.begin) + ", " + std::to_string(t.end) +
                           ") lies outside the " + std::to_string(f->data_len_) + " data bytes");
        // the product of the sizes, refusing what would not fit 63 bits
        uint64_t need = (uint64_t)esize;
        bool overflow = false;
        for (int64_t d : t.shape) {
            if (d != 0 && need > (uint64_t)INT64_MAX / (uint64_t)d) { overflow = true; break; }
            need *= (uint64_t)d;
        }
        if (overflow || need != (uint64_t)(t.end - t.begin))
            return give_up("tensor " + quoted(name) + " of shape " + shape_text(t.shape) + " " + t.dtype + " needs " +
                           (overflow ? std::string("more than 2^63") : std::to_string(need)) + " bytes, has " +
                           std::to_string(t.end - t.begin));
        f->tensors_.push_back(std::move(t));
    }
    return f;
}

}  // namespace allpaca
