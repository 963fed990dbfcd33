#include <cctype>
#include <cmath>
#include <cstdlib>
#include <sstream>

#include <stdml/bits/collective/json.hpp>

namespace stdml::collective::json
{
value value::boolean(bool b)
{
    value v;
    v.kind_ = bool_k;
    v.bool_ = b;
    return v;
}

value value::number(double d)
{
    value v;
    v.kind_ = number_k;
    v.num_ = d;
    return v;
}

value value::integer(int64_t i)
{
    value v;
    v.kind_ = number_k;
    v.is_int_ = true;
    v.int_ = i;
    v.num_ = static_cast<double>(i);
    return v;
}

value value::string(std::string s)
{
    value v;
    v.kind_ = string_k;
    v.str_ = std::move(s);
    return v;
}

value value::array(std::vector<value> xs)
{
    value v;
    v.kind_ = array_k;
    v.arr_ = std::move(xs);
    return v;
}

value value::object(std::vector<std::pair<std::string, value>> kv)
{
    value v;
    v.kind_ = object_k;
    v.obj_ = std::move(kv);
    return v;
}

const value *value::get(const std::string &key) const
{
    if (kind_ != object_k) { return nullptr; }
    for (const auto &kv : obj_) {
        if (kv.first == key) { return &kv.second; }
    }
    return nullptr;
}

void value::set(const std::string &key, value v)
{
    kind_ = object_k;
    for (auto &kv : obj_) {
        if (kv.first == key) {
            kv.second = std::move(v);
            return;
        }
    }
    obj_.emplace_back(key, std::move(v));
}

std::string quote(const std::string &s)
{
    std::string out = "\"";
    for (unsigned char c : s) {
        switch (c) {
        case '"':
            out += "\\\"";
            break;
        case '\\':
            out += "\\\\";
            break;
        case '\n':
            out += "\\n";
            break;
        case '\r':
            out += "\\r";
            break;
        case '\t':
            out += "\\t";
            break;
        default:
            if (c < 0x20) {
                char buf[8];
                std::snprintf(buf, sizeof(buf), "\\u%04x", c);
                out += buf;
            } else {
                out += static_cast<char>(c);
            }
        }
    }
    out += '"';
    return out;
}

std::string to_json(const std::string &s) { return quote(s); }
std::string to_json(int64_t i) { return std::to_string(i); }

std::string value::dump() const
{
    switch (kind_) {
    case null_k:
        return "null";
    case bool_k:
        return bool_ ? "true" : "false";
    case number_k: {
        if (is_int_) { return std::to_string(int_); }
        if (std::floor(num_) == num_ && std::fabs(num_) < 9e15) {
            return std::to_string(static_cast<int64_t>(num_));
        }
        std::ostringstream ss;
        ss.precision(17);
        ss << num_;
        return ss.str();
    }
    case string_k:
        return quote(str_);
    case array_k: {
        std::string out = "[";
        for (size_t i = 0; i < arr_.size(); ++i) {
            if (i) { out += ','; }
            out += arr_[i].dump();
        }
        return out + "]";
    }
    case object_k: {
        std::string out = "{";
        for (size_t i = 0; i < obj_.size(); ++i) {
            if (i) { out += ','; }
            out += quote(obj_[i].first) + ":" + obj_[i].second.dump();
        }
        return out + "}";
    }
    }
    return "null";
}

namespace
{
struct reader {
    const std::string &s;
    size_t i = 0;
    int depth = 0;

    void ws()
    {
        while (i < s.size() && std::isspace(static_cast<unsigned char>(s[i]))) { ++i; }
    }

    bool lit(const char *w)
    {
        const size_t n = std::char_traits<char>::length(w);
        if (s.compare(i, n, w) == 0) {
            i += n;
            return true;
        }
        return false;
    }

    static void utf8(std::string &out, uint32_t cp)
    {
        if (cp < 0x80) {
            out += static_cast<char>(cp);
        } else if (cp < 0x800) {
            out += static_cast<char>(0xc0 | (cp >> 6));
            out += static_cast<char>(0x80 | (cp & 0x3f));
        } else if (cp < 0x10000) {
            out += static_cast<char>(0xe0 | (cp >> 12));
            out += static_cast<char>(0x80 | ((cp >> 6) & 0x3f));
            out += static_cast<char>(0x80 | (cp & 0x3f));
        } else {
            out += static_cast<char>(0xf0 | (cp >> 18));
            out += static_cast<char>(0x80 | ((cp >> 12) & 0x3f));
            out += static_cast<char>(0x80 | ((cp >> 6) & 0x3f));
            out += static_cast<char>(0x80 | (cp & 0x3f));
        }
    }

    bool hex4(uint32_t &cp)
    {
        if (i + 4 > s.size()) { return false; }
        cp = 0;
        for (int k = 0; k < 4; ++k) {
            const char c = s[i++];
            cp <<= 4;
            if (c >= '0' && c <= '9') {
                cp |= c - '0';
            } else if (c >= 'a' && c <= 'f') {
                cp |= c - 'a' + 10;
            } else if (c >= 'A' && c <= 'F') {
                cp |= c - 'A' + 10;
            } else {
                return false;
            }
        }
        return true;
    }

    bool str(std::string &out)
    {
        if (i >= s.size() || s[i] != '"') { return false; }
        ++i;
        while (i < s.size()) {
            const char c = s[i++];
            if (c == '"') { return true; }
            if (c != '\\') {
                out += c;
                continue;
            }
            if (i >= s.size()) { return false; }
            const char e = s[i++];
            switch (e) {
            case '"':
            case '\\':
            case '/':
                out += e;
                break;
            case 'b':
                out += '\b';
                break;
            case 'f':
                out += '\f';
                break;
            case 'n':
                out += '\n';
                break;
            case 'r':
                out += '\r';
                break;
            case 't':
                out += '\t';
                break;
            case 'u': {
                uint32_t cp;
                if (!hex4(cp)) { return false; }
                if (cp >= 0xd800 && cp < 0xdc00 && s.compare(i, 2, "\\u") == 0) {
                    i += 2;
                    uint32_t lo;
                    if (!hex4(lo)) { return false; }
                    cp = 0x10000 + ((cp - 0xd800) << 10) + (lo - 0xdc00);
                }
                utf8(out, cp);
                break;
            }
            default:
                return false;
            }
        }
        return false;
    }

    bool val(value &out)
    {
        if (++depth > 256) { return false; }
        ws();
        if (i >= s.size()) { return false; }
        bool ok = false;
        const char c = s[i];
        if (c == '{') {
            ++i;
            out = value::object();
            ws();
            if (i < s.size() && s[i] == '}') {
                ++i;
                ok = true;
            } else {
                for (;;) {
                    ws();
                    std::string k;
                    value v;
                    if (!str(k)) { break; }
                    ws();
                    if (i >= s.size() || s[i++] != ':') { break; }
                    if (!val(v)) { break; }
                    out.set(k, std::move(v));
                    ws();
                    if (i < s.size() && s[i] == ',') {
                        ++i;
                        continue;
                    }
                    if (i < s.size() && s[i] == '}') {
                        ++i;
                        ok = true;
                    }
                    break;
                }
            }
        } else if (c == '[') {
            ++i;
            out = value::array();
            ws();
            if (i < s.size() && s[i] == ']') {
                ++i;
                ok = true;
            } else {
                for (;;) {
                    value v;
                    if (!val(v)) { break; }
                    out.push(std::move(v));
                    ws();
                    if (i < s.size() && s[i] == ',') {
                        ++i;
                        continue;
                    }
                    if (i < s.size() && s[i] == ']') {
                        ++i;
                        ok = true;
                    }
                    break;
                }
            }
        } else if (c == '"') {
            std::string t;
            ok = str(t);
            if (ok) { out = value::string(std::move(t)); }
        } else if (lit("true")) {
            out = value::boolean(true);
            ok = true;
        } else if (lit("false")) {
            out = value::boolean(false);
            ok = true;
        } else if (lit("null")) {
            out = value();
            ok = true;
        } else {
            const size_t start = i;
            if (i < s.size() && (s[i] == '-' || s[i] == '+')) { ++i; }
            bool digits = false, frac = false;
            while (i < s.size()) {
                const char d = s[i];
                if (std::isdigit(static_cast<unsigned char>(d))) {
                    digits = true;
                } else if (d == '.' || d == 'e' || d == 'E' || d == '-' || d == '+') {
                    frac = true;
                } else {
                    break;
                }
                ++i;
            }
            if (digits) {
                const std::string tok = s.substr(start, i - start);
                if (!frac) {
                    errno = 0;
                    const long long n = std::strtoll(tok.c_str(), nullptr, 10);
                    if (errno == 0) {
                        out = value::integer(n);
                    } else {
                        out = value::number(std::strtod(tok.c_str(), nullptr));
                    }
                } else {
                    out = value::number(std::strtod(tok.c_str(), nullptr));
                }
                ok = true;
            }
        }
        --depth;
        return ok;
    }
};
}  // namespace

std::optional<value> parse(const std::string &text)
{
    reader r{text};
    value v;
    if (!r.val(v)) { return {}; }
    r.ws();
    if (r.i != text.size()) { return {}; }
    return v;
}
}  // namespace stdml::collective::json
