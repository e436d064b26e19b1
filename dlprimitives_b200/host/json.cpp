// JSON document model: parser and writer.
#include <dlprim/json.hpp>
#include <cmath>
#include <cstdlib>
#include <limits>
#include <sstream>
#include <cstring>
#include <cstdio>
#include <cctype>

namespace dlprim {
namespace json {

value::value(value const &o) : type_(o.type_), b_(o.b_), n_(o.n_), s_(o.s_)
{
    if(o.a_) a_.reset(new json::array(*o.a_));
    if(o.o_) o_.reset(new json::object(*o.o_));
}
value &value::operator=(value const &o)
{
    if(this != &o) {
        value tmp(o);
        *this = std::move(tmp);
    }
    return *this;
}

static char const *type_name(json_type t)
{
    static char const *names[] = {"undefined", "null", "boolean", "number", "string", "object", "array"};
    return names[int(t)];
}
static bad_value_cast wrong(char const *want, json_type got)
{
    return bad_value_cast(std::string("expected ") + want + ", got " + type_name(got));
}

bool value::boolean() const { if(type_ != is_boolean) throw wrong("boolean", type_); return b_; }
double value::number() const { if(type_ != is_number) throw wrong("number", type_); return n_; }
std::string const &value::str() const { if(type_ != is_string) throw wrong("string", type_); return s_; }
json::array const &value::array() const { if(type_ != is_array) throw wrong("array", type_); return *a_; }
json::array &value::array()
{
    if(type_ == json::is_undefined) { type_ = is_array; a_.reset(new json::array()); }
    if(type_ != is_array) throw wrong("array", type_);
    return *a_;
}
json::object const &value::object() const { if(type_ != is_object) throw wrong("object", type_); return *o_; }
json::object &value::object()
{
    if(type_ == json::is_undefined) { type_ = is_object; o_.reset(new json::object()); }
    if(type_ != is_object) throw wrong("object", type_);
    return *o_;
}

value const &value::find(std::string const &path) const
{
    static const value undefined;
    value const *cur = this;
    size_t pos = 0;
    while(true) {
        if(cur->type_ != is_object) return undefined;
        size_t dot = path.find('.', pos);
        // a key that itself contains dots wins over path splitting
        auto whole = cur->o_->find(path.substr(pos));
        if(whole != cur->o_->end()) return whole->second;
        std::string key = path.substr(pos, dot == std::string::npos ? std::string::npos : dot - pos);
        auto it = cur->o_->find(key);
        if(it == cur->o_->end()) return undefined;
        cur = &it->second;
        if(dot == std::string::npos) return *cur;
        pos = dot + 1;
    }
}
value const &value::at(std::string const &path) const
{
    value const &v = find(path);
    if(v.is_undefined()) throw bad_value_cast("missing member " + path);
    return v;
}
value &value::operator[](std::string const &key) { return object()[key]; }

template<> bool value::get_value<bool>() const { return boolean(); }
template<> double value::get_value<double>() const { return number(); }
template<> float value::get_value<float>() const { return float(number()); }
template<> int value::get_value<int>() const
{
    double v = number();
    if(v != std::floor(v) || v < std::numeric_limits<int>::min() || v > std::numeric_limits<int>::max())
        throw bad_value_cast("number is not an int");
    return int(v);
}
template<> unsigned value::get_value<unsigned>() const
{
    double v = number();
    if(v != std::floor(v) || v < 0 || v > std::numeric_limits<unsigned>::max()) throw bad_value_cast("number is not an unsigned int");
    return unsigned(v);
}
template<> size_t value::get_value<size_t>() const
{
    double v = number();
    if(v != std::floor(v) || v < 0) throw bad_value_cast("number is not a size");
    return size_t(v);
}
template<> std::string value::get_value<std::string>() const { return str(); }
template<> std::vector<int> value::get_value<std::vector<int> >() const
{
    std::vector<int> r;
    for(value const &v : array()) r.push_back(v.get_value<int>());
    return r;
}
template<> std::vector<float> value::get_value<std::vector<float> >() const
{
    std::vector<float> r;
    for(value const &v : array()) r.push_back(v.get_value<float>());
    return r;
}
template<> std::vector<std::string> value::get_value<std::vector<std::string> >() const
{
    std::vector<std::string> r;
    for(value const &v : array()) r.push_back(v.str());
    return r;
}

// ------------------------------------------------------------------------------------------ parser
namespace {
struct Parser {
    char const *p, *end;
    int line = 1;
    bool ok = true;

    void skip()
    {
        while(p < end) {
            if(*p == '\n') { line++; p++; }
            else if(*p == ' ' || *p == '\t' || *p == '\r') p++;
            else if(*p == '/' && p + 1 < end && p[1] == '/') { while(p < end && *p != '\n') p++; }
            else break;
        }
    }
    bool lit(char const *s)
    {
        size_t n = strlen(s);
        if(size_t(end - p) >= n && std::char_traits<char>::compare(p, s, n) == 0) { p += n; return true; }
        return false;
    }
    static void utf8(std::string &out, unsigned cp)
    {
        if(cp < 0x80) out += char(cp);
        else if(cp < 0x800) { out += char(0xC0 | (cp >> 6)); out += char(0x80 | (cp & 0x3F)); }
        else if(cp < 0x10000) { out += char(0xE0 | (cp >> 12)); out += char(0x80 | ((cp >> 6) & 0x3F)); out += char(0x80 | (cp & 0x3F)); }
        else { out += char(0xF0 | (cp >> 18)); out += char(0x80 | ((cp >> 12) & 0x3F)); out += char(0x80 | ((cp >> 6) & 0x3F)); out += char(0x80 | (cp & 0x3F)); }
    }
    bool hex4(unsigned &v)
    {
        if(end - p < 4) return false;
        v = 0;
        for(int i = 0; i < 4; i++, p++) {
            char c = *p;
            v <<= 4;
            if(c >= '0' && c <= '9') v |= c - '0';
            else if(c >= 'a' && c <= 'f') v |= c - 'a' + 10;
            else if(c >= 'A' && c <= 'F') v |= c - 'A' + 10;
            else return false;
        }
        return true;
    }
    bool string(std::string &out)
    {
        if(p >= end || *p != '"') return false;
        p++;
        while(p < end && *p != '"') {
            if(*p == '\\') {
                if(++p >= end) return false;
                switch(*p++) {
                case '"': out += '"'; break;
                case '\\': out += '\\'; break;
                case '/': out += '/'; break;
                case 'b': out += '\b'; break;
                case 'f': out += '\f'; break;
                case 'n': out += '\n'; break;
                case 'r': out += '\r'; break;
                case 't': out += '\t'; break;
                case 'u': {
                    unsigned cp;
                    if(!hex4(cp)) return false;
                    if(cp >= 0xD800 && cp < 0xDC00 && end - p >= 6 && p[0] == '\\' && p[1] == 'u') {
                        p += 2;
                        unsigned lo;
                        if(!hex4(lo)) return false;
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    utf8(out, cp);
                    break;
                }
                default: return false;
                }
            }
            else {
                if(*p == '\n') line++;
                out += *p++;
            }
        }
        if(p >= end) return false;
        p++;
        return true;
    }
    bool parse(value &v, int depth)
    {
        if(depth > 200) return false;
        skip();
        if(p >= end) return false;
        char c = *p;
        if(c == '{') {
            p++;
            json::object &o = v.object();
            skip();
            if(p < end && *p == '}') { p++; return true; }
            while(true) {
                skip();
                std::string key;
                if(!string(key)) return false;
                skip();
                if(p >= end || *p != ':') return false;
                p++;
                if(!parse(o[key], depth + 1)) return false;
                skip();
                if(p < end && *p == ',') { p++; continue; }
                if(p < end && *p == '}') { p++; return true; }
                return false;
            }
        }
        if(c == '[') {
            p++;
            json::array &a = v.array();
            skip();
            if(p < end && *p == ']') { p++; return true; }
            while(true) {
                a.push_back(value());
                if(!parse(a.back(), depth + 1)) return false;
                skip();
                if(p < end && *p == ',') { p++; continue; }
                if(p < end && *p == ']') { p++; return true; }
                return false;
            }
        }
        if(c == '"') {
            std::string s;
            if(!string(s)) return false;
            v = value(s);
            return true;
        }
        if(lit("true")) { v = value(true); return true; }
        if(lit("false")) { v = value(false); return true; }
        if(lit("null")) { v.null(); return true; }
        if(c == '-' || (c >= '0' && c <= '9')) {
            std::string num;
            while(p < end && (std::isdigit((unsigned char)*p) || *p == '-' || *p == '+' || *p == '.' || *p == 'e' || *p == 'E')) num += *p++;
            char *stop = nullptr;
            double d = std::strtod(num.c_str(), &stop);
            if(!stop || *stop != 0) return false;
            v = value(d);
            return true;
        }
        return false;
    }
};
} // namespace

bool value::load(char const *&begin, char const *end, bool full, int *line_number)
{
    Parser ps{begin, end};
    value tmp;
    bool ok = ps.parse(tmp, 0);
    if(ok && full) {
        ps.skip();
        ok = ps.p == end;
    }
    if(line_number) *line_number = ps.line;
    begin = ps.p;
    if(ok) *this = std::move(tmp);
    return ok;
}
bool value::load(std::istream &in, bool full, int *line_number)
{
    std::ostringstream ss;
    ss << in.rdbuf();
    std::string text = ss.str();
    char const *b = text.c_str();
    return load(b, b + text.size(), full, line_number);
}
value parse(std::string const &text)
{
    value v;
    char const *b = text.c_str();
    int line = 0;
    if(!v.load(b, b + text.size(), true, &line)) throw ValidationError("JSON syntax error near line " + std::to_string(line));
    return v;
}

// ------------------------------------------------------------------------------------------ writer
static void write_string(std::ostream &out, std::string const &s)
{
    out << '"';
    for(unsigned char c : s) {
        switch(c) {
        case '"': out << "\\\""; break;
        case '\\': out << "\\\\"; break;
        case '\n': out << "\\n"; break;
        case '\r': out << "\\r"; break;
        case '\t': out << "\\t"; break;
        default:
            if(c < 0x20) { char buf[8]; snprintf(buf, sizeof(buf), "\\u%04x", c); out << buf; }
            else out << char(c);
        }
    }
    out << '"';
}
void value::write(std::ostream &out, int how, int indent) const
{
    auto nl = [&](int ind) { if(how == readable) { out << '\n'; for(int i = 0; i < ind; i++) out << "  "; } };
    switch(type_) {
    case json::is_undefined: case json::is_null: out << "null"; break;
    case is_boolean: out << (b_ ? "true" : "false"); break;
    case is_number: {
        if(n_ == std::floor(n_) && std::fabs(n_) < 1e15) out << (long long)n_;
        else { std::ostringstream ss; ss.precision(17); ss << n_; out << ss.str(); }
        break;
    }
    case is_string: write_string(out, s_); break;
    case is_array: {
        out << '[';
        bool first = true;
        for(value const &v : *a_) { if(!first) out << ','; first = false; nl(indent + 1); v.write(out, how, indent + 1); }
        if(!a_->empty()) nl(indent);
        out << ']';
        break;
    }
    case is_object: {
        out << '{';
        bool first = true;
        for(auto const &kv : *o_) {
            if(!first) out << ',';
            first = false;
            nl(indent + 1);
            write_string(out, kv.first);
            out << ':';
            kv.second.write(out, how, indent + 1);
        }
        if(!o_->empty()) nl(indent);
        out << '}';
        break;
    }
    }
}
void value::save(std::ostream &out, int how) const { write(out, how, 0); }
std::string value::save(int how) const
{
    std::ostringstream ss;
    save(ss, how);
    return ss.str();
}

} // namespace json
} // namespace dlprim
