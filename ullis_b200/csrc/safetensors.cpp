#include "safetensors.hpp"

#include <cstdlib>
#include <cstring>

#include "common.hpp"

namespace ullis {

namespace {

struct Parser {
    const char* p;
    const char* end;

    [[noreturn]] void bad(const char* what) { fail(ULLIS_CUDA_ERR_CHECKPOINT, std::string("JSON: ") + what); }
    void ws() {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
    }
    bool eat(char c) {
        ws();
        if (p < end && *p == c) {
            ++p;
            return true;
        }
        return false;
    }
    void append_utf8(std::string& out, uint32_t cp) {
        if (cp < 0x80) {
            out += (char)cp;
        } else if (cp < 0x800) {
            out += (char)(0xC0 | (cp >> 6));
            out += (char)(0x80 | (cp & 0x3F));
        } else if (cp < 0x10000) {
            out += (char)(0xE0 | (cp >> 12));
            out += (char)(0x80 | ((cp >> 6) & 0x3F));
            out += (char)(0x80 | (cp & 0x3F));
        } else {
            out += (char)(0xF0 | (cp >> 18));
            out += (char)(0x80 | ((cp >> 12) & 0x3F));
            out += (char)(0x80 | ((cp >> 6) & 0x3F));
            out += (char)(0x80 | (cp & 0x3F));
        }
    }
    uint32_t hex4() {
        if (end - p < 4) bad("truncated \\u escape");
        uint32_t v = 0;
        for (int i = 0; i < 4; ++i) {
            char c = *p++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= (uint32_t)(c - '0');
            else if (c >= 'a' && c <= 'f') v |= (uint32_t)(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= (uint32_t)(c - 'A' + 10);
            else bad("bad \\u escape");
        }
        return v;
    }
    std::string string() {
        ws();
        if (p >= end || *p != '"') bad("expected string");
        ++p;
        std::string out;
        while (true) {
            if (p >= end) bad("unterminated string");
            char c = *p++;
            if (c == '"') break;
            if (c == '\\') {
                if (p >= end) bad("unterminated escape");
                char e = *p++;
                switch (e) {
                    case '"': out += '"'; break;
                    case '\\': out += '\\'; break;
                    case '/': out += '/'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'n': out += '\n'; break;
                    case 'r': out += '\r'; break;
                    case 't': out += '\t'; break;
                    case 'u': {
                        uint32_t cp = hex4();
                        if (cp >= 0xD800 && cp < 0xDC00 && end - p >= 6 && p[0] == '\\' && p[1] == 'u') {
                            p += 2;
                            uint32_t lo = hex4();
                            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                        }
                        append_utf8(out, cp);
                        break;
                    }
                    default: bad("unknown escape");
                }
            } else {
                out += c;
            }
        }
        return out;
    }
    Json value(int depth) {
        if (depth > 32) bad("nesting too deep");
        ws();
        if (p >= end) bad("unexpected end");
        Json j;
        char c = *p;
        if (c == '{') {
            ++p;
            j.kind = Json::Object;
            if (eat('}')) return j;
            do {
                std::string key = string();
                if (!eat(':')) bad("expected ':'");
                j.members.emplace_back(std::move(key), value(depth + 1));
            } while (eat(','));
            if (!eat('}')) bad("expected '}'");
        } else if (c == '[') {
            ++p;
            j.kind = Json::Array;
            if (eat(']')) return j;
            do {
                j.items.push_back(value(depth + 1));
            } while (eat(','));
            if (!eat(']')) bad("expected ']'");
        } else if (c == '"') {
            j.kind = Json::String;
            j.text = string();
        } else if (c == 't' && end - p >= 4 && !strncmp(p, "true", 4)) {
            p += 4;
            j.kind = Json::Bool;
            j.boolean = true;
        } else if (c == 'f' && end - p >= 5 && !strncmp(p, "false", 5)) {
            p += 5;
            j.kind = Json::Bool;
        } else if (c == 'n' && end - p >= 4 && !strncmp(p, "null", 4)) {
            p += 4;
        } else if (c == '-' || (c >= '0' && c <= '9')) {
            const char* s = p;
            while (p < end && (*p == '-' || *p == '+' || *p == '.' || *p == 'e' || *p == 'E' ||
                               (*p >= '0' && *p <= '9')))
                ++p;
            j.kind = Json::Number;
            j.text.assign(s, p);
            j.number = strtod(j.text.c_str(), nullptr);
        } else {
            bad("unexpected character");
        }
        return j;
    }
};

}  // namespace

const Json* Json::get(const std::string& key) const {
    for (const auto& m : members)
        if (m.first == key) return &m.second;
    return nullptr;
}

uint64_t Json::u64(const std::string& key, uint64_t fallback, bool* present) const {
    const Json* j = get(key);
    if (present) *present = j && j->kind == Number;
    if (!j || j->kind != Number) return fallback;
    if (j->text.find_first_of(".eE-") != std::string::npos) {
        if (j->number < 0) fail(ULLIS_CUDA_ERR_CHECKPOINT, "config field " + key + " must be a non-negative integer");
        return (uint64_t)j->number;
    }
    return strtoull(j->text.c_str(), nullptr, 10);
}

Json parse_json(const char* data, size_t len) {
    Parser ps{data, data + len};
    Json j = ps.value(0);
    ps.ws();
    if (ps.p != ps.end) ps.bad("trailing characters");
    return j;
}

size_t TensorView::elements() const {
    if (dtype == "F16" || dtype == "BF16" || dtype == "I16" || dtype == "U16") return bytes / 2;
    if (dtype == "F32" || dtype == "U32" || dtype == "I32") return bytes / 4;
    if (dtype == "F64" || dtype == "U64" || dtype == "I64") return bytes / 8;
    return bytes;
}

SafeTensors parse_safetensors(const uint8_t* bytes, size_t len) {
    if (!bytes || len < 8) fail(ULLIS_CUDA_ERR_CHECKPOINT, "parse safetensors checkpoint header: file too short");
    uint64_t hlen = 0;
    for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | bytes[i];
    if (hlen > len - 8 || hlen > ((uint64_t)100 << 20))
        fail(ULLIS_CUDA_ERR_CHECKPOINT, "parse safetensors checkpoint header: bad header length");
    Json header = parse_json(reinterpret_cast<const char*>(bytes + 8), (size_t)hlen);
    if (header.kind != Json::Object)
        fail(ULLIS_CUDA_ERR_CHECKPOINT, "parse safetensors checkpoint header: not a JSON object");
    const uint8_t* base = bytes + 8 + hlen;
    const size_t data_len = len - 8 - (size_t)hlen;
    SafeTensors st;
    for (const auto& m : header.members) {
        if (m.first == "__metadata__") {
            if (m.second.kind != Json::Object)
                fail(ULLIS_CUDA_ERR_CHECKPOINT, "parse safetensors checkpoint header: bad metadata");
            st.has_metadata = true;
            for (const auto& kv : m.second.members)
                if (kv.second.kind == Json::String) st.metadata[kv.first] = kv.second.text;
            continue;
        }
        const Json* dt = m.second.get("dtype");
        const Json* off = m.second.get("data_offsets");
        if (m.second.kind != Json::Object || !dt || dt->kind != Json::String || !off || off->kind != Json::Array ||
            off->items.size() != 2)
            fail(ULLIS_CUDA_ERR_CHECKPOINT, "parse safetensors checkpoint: bad entry for tensor " + m.first);
        const uint64_t b = (uint64_t)off->items[0].number, e = (uint64_t)off->items[1].number;
        if (b > e || e > data_len)
            fail(ULLIS_CUDA_ERR_CHECKPOINT, "parse safetensors checkpoint: tensor " + m.first + " out of bounds");
        TensorView v;
        v.dtype = dt->text;
        v.data = base + b;
        v.bytes = (size_t)(e - b);
        st.tensors[m.first] = v;
    }
    return st;
}

}  // namespace ullis
