// Minimal stand-in for the part of {fmt} the reference's benchmarks use: fmt::print / fmt::format with "{}"
// and printf-like specs such as "{:.3f}", "{:10.3f}", "{:>8}", "{:<12}", "{:d}". Written for this repository (the
// {fmt} library is not installed here); not a general implementation.
#pragma once
#include <cstdio>
#include <sstream>
#include <string>
#include <string_view>
#include <type_traits>

namespace fmt {
namespace detail {

template <typename T>
std::string format_one(std::string_view spec, const T& value) {
    // spec: [[fill]align][width][.precision][type]
    char align = 0;
    size_t i = 0;
    if (spec.size() >= 1 && (spec[0] == '<' || spec[0] == '>' || spec[0] == '^')) align = spec[i++];
    int width = 0, precision = -1;
    while (i < spec.size() && spec[i] >= '0' && spec[i] <= '9') width = width * 10 + (spec[i++] - '0');
    if (i < spec.size() && spec[i] == '.') {
        ++i;
        precision = 0;
        while (i < spec.size() && spec[i] >= '0' && spec[i] <= '9') precision = precision * 10 + (spec[i++] - '0');
    }
    const char type = i < spec.size() ? spec[i] : 0;
    std::string body;
    if constexpr (std::is_floating_point_v<T>) {
        char buf[128];
        if (precision >= 0 || type == 'f' || type == 'e' || type == 'g') {
            const char conv = (type == 'e' || type == 'g') ? type : 'f';
            const char f[] = {'%', '.', '*', conv, 0};
            std::snprintf(buf, sizeof(buf), f, precision < 0 ? 6 : precision, static_cast<double>(value));
        } else {
            std::snprintf(buf, sizeof(buf), "%g", static_cast<double>(value));
        }
        body = buf;
        if (!align) align = '>';
    } else if constexpr (std::is_integral_v<T> && !std::is_same_v<T, bool> && !std::is_same_v<T, char>) {
        body = std::to_string(value);
        if (!align) align = '>';
    } else {
        std::ostringstream os;
        os << value;
        body = os.str();
        if (!align) align = '<';
    }
    if (static_cast<int>(body.size()) < width) {
        const size_t pad = static_cast<size_t>(width) - body.size();
        if (align == '>')
            body.insert(0, pad, ' ');
        else if (align == '^')
            body = std::string(pad / 2, ' ') + body + std::string(pad - pad / 2, ' ');
        else
            body.append(pad, ' ');
    }
    return body;
}

inline void format_rest(std::string& out, std::string_view f) {
    for (size_t i = 0; i < f.size(); ++i) {
        if ((f[i] == '{' || f[i] == '}') && i + 1 < f.size() && f[i + 1] == f[i]) ++i;
        out.push_back(f[i]);
    }
}

template <typename T, typename... Rest>
void format_rest(std::string& out, std::string_view f, const T& first, const Rest&... rest) {
    for (size_t i = 0; i < f.size(); ++i) {
        if (f[i] == '{' && i + 1 < f.size() && f[i + 1] == '{') {
            out.push_back('{');
            ++i;
        } else if (f[i] == '}' && i + 1 < f.size() && f[i + 1] == '}') {
            out.push_back('}');
            ++i;
        } else if (f[i] == '{') {
            const size_t close = f.find('}', i);
            if (close == std::string_view::npos) break;
            std::string_view spec = f.substr(i + 1, close - i - 1);
            const size_t colon = spec.find(':');
            spec = colon == std::string_view::npos ? std::string_view{} : spec.substr(colon + 1);
            out += format_one(spec, first);
            format_rest(out, f.substr(close + 1), rest...);
            return;
        } else {
            out.push_back(f[i]);
        }
    }
}

}  // namespace detail

template <typename... Args>
std::string format(std::string_view f, const Args&... args) {
    std::string out;
    detail::format_rest(out, f, args...);
    return out;
}

template <typename... Args>
void print(std::string_view f, const Args&... args) {
    const std::string s = format(f, args...);
    std::fwrite(s.data(), 1, s.size(), stdout);
}

template <typename... Args>
void print(std::FILE* file, std::string_view f, const Args&... args) {
    const std::string s = format(f, args...);
    std::fwrite(s.data(), 1, s.size(), file);
}

}  // namespace fmt
