// A small JSON document model: enough to read the network / operator-option schema the reference
// documents in docs/network_json_format.md (objects, arrays, strings, numbers, booleans, null) and
// to write it back.  The accessor names follow the reference's json::value (include/dlprim/json.hpp)
// where Net and the operators use them: get<T>(path), get(path, default), find(path), operator[],
// array(), object(), str(), number(), boolean(), load(), save().  Paths may be dotted ("a.b").
#pragma once
#include <dlprim/definitions.hpp>
#include <istream>
#include <map>
#include <memory>
#include <ostream>
#include <string>
#include <type_traits>
#include <vector>

namespace dlprim {
namespace json {

    class DLPRIM_API bad_value_cast : public ValidationError {
    public:
        explicit bad_value_cast(std::string const &m) : ValidationError("json: " + m) {}
    };

    enum json_type { is_undefined, is_null, is_boolean, is_number, is_string, is_object, is_array };
    enum { compact = 0, readable = 1 };

    class value;
    typedef std::vector<value> array;
    typedef std::map<std::string, value> object;

    class DLPRIM_API value {
    public:
        value() : type_(json::is_undefined), b_(false), n_(0) {}
        value(bool v) : type_(is_boolean), b_(v), n_(0) {}
        value(int v) : type_(is_number), b_(false), n_(v) {}
        value(double v) : type_(is_number), b_(false), n_(v) {}
        value(char const *s) : type_(is_string), b_(false), n_(0), s_(s) {}
        value(std::string const &s) : type_(is_string), b_(false), n_(0), s_(s) {}
        value(json::array const &a) : type_(is_array), b_(false), n_(0), a_(new json::array(a)) {}
        value(json::object const &o) : type_(is_object), b_(false), n_(0), o_(new json::object(o)) {}
        value(value const &other);
        value &operator=(value const &other);
        value(value &&) = default;
        value &operator=(value &&) = default;

        json_type type() const { return type_; }
        bool is_undefined() const { return type_ == json::is_undefined; }
        bool is_null() const { return type_ == json::is_null; }
        void null() { *this = value(); type_ = json::is_null; }

        bool boolean() const;
        double number() const;
        std::string const &str() const;
        json::array const &array() const;
        json::array &array();
        json::object const &object() const;
        json::object &object();

        /// Member lookup by (dotted) path; an undefined value when absent.
        value const &find(std::string const &path) const;
        /// Member lookup that throws when absent.
        value const &at(std::string const &path) const;
        value const &operator[](std::string const &path) const { return at(path); }
        value const &operator[](char const *path) const { return at(path); }
        /// Creates the member (and the object) when absent.
        value &operator[](std::string const &key);
        value &operator[](char const *key) { return (*this)[std::string(key)]; }
        value const &operator[](size_t i) const { return array().at(i); }

        template<typename T> T get_value() const;
        template<typename T> T get(std::string const &path) const { return at(path).get_value<T>(); }
        /// The default also stands in when the member exists but cannot be converted to T, as in the reference
        /// (include/dlprim/json.hpp:918-950): its own network files write booleans as 0 / 1 in places.
        template<typename T> T get(std::string const &path, T const &def) const
        {
            value const &v = find(path);
            if(v.is_undefined()) return def;
            try {
                return v.get_value<T>();
            }
            catch(bad_value_cast const &) {
                return def;
            }
        }
        std::string get(std::string const &path, char const *def) const { return get<std::string>(path, std::string(def)); }

        /// Parse a whole document; returns false (and the line) on a syntax error.
        bool load(std::istream &in, bool full, int *line_number = nullptr);
        bool load(char const *&begin, char const *end, bool full, int *line_number = nullptr);
        void save(std::ostream &out, int how = compact) const;
        std::string save(int how = compact) const;

    private:
        void write(std::ostream &out, int how, int indent) const;
        json_type type_;
        bool b_;
        double n_;
        std::string s_;
        std::unique_ptr<json::array> a_;
        std::unique_ptr<json::object> o_;
    };

    template<> DLPRIM_API bool value::get_value<bool>() const;
    template<> DLPRIM_API int value::get_value<int>() const;
    template<> DLPRIM_API unsigned value::get_value<unsigned>() const;
    template<> DLPRIM_API size_t value::get_value<size_t>() const;
    template<> DLPRIM_API float value::get_value<float>() const;
    template<> DLPRIM_API double value::get_value<double>() const;
    template<> DLPRIM_API std::string value::get_value<std::string>() const;
    template<> DLPRIM_API std::vector<int> value::get_value<std::vector<int> >() const;
    template<> DLPRIM_API std::vector<float> value::get_value<std::vector<float> >() const;
    template<> DLPRIM_API std::vector<std::string> value::get_value<std::vector<std::string> >() const;

    /// Parse text; throws ValidationError on a syntax error.
    DLPRIM_API value parse(std::string const &text);

} // namespace json

namespace utils {
    /// Options such as "kernel": 3 or "kernel": [3,5] (the reference's get_1dNd_from_json,
    /// include/dlprim/utils/json_helpers.hpp:27-49).
    template<size_t N>
    void get_1dNd_from_json(json::value const &v, std::string const &name, int (&vals)[N], bool required = false)
    {
        json::value const &m = v.find(name);
        if(m.is_undefined()) {
            if(required) throw ValidationError("Missing required option " + name);
            return;
        }
        if(m.type() == json::is_array) {
            std::vector<int> a = m.get_value<std::vector<int> >();
            if(a.size() != N) throw ValidationError("Option " + name + " has a wrong number of values");
            for(size_t i = 0; i < N; i++) vals[i] = a[i];
        }
        else {
            int s = m.get_value<int>();
            for(size_t i = 0; i < N; i++) vals[i] = s;
        }
    }
}
} // namespace dlprim
