#pragma once
// Test infrastructure only. Stand-ins for the few Boost facilities that the reference's
// layer sources name, so that those sources compile in an image without Boost headers.
// Everything maps onto the C++ standard library.
#include <memory>
#include <random>
#include <sstream>
#include <string>
#include <vector>
namespace boost {
typedef std::mt19937 mt19937;
template <class T> using normal_distribution = std::normal_distribution<T>;
namespace random {
template <class T> using uniform_real_distribution = std::uniform_real_distribution<T>;
template <class T> using normal_distribution = std::normal_distribution<T>;
}  // namespace random
struct any_of_set { std::string chars; };
inline any_of_set is_any_of(const std::string &s) { any_of_set a; a.chars = s; return a; }
inline void split(std::vector<std::string> &out, const std::string &in, const any_of_set &d) {
    out.clear();
    std::string cur;
    for (char c : in) {
        if (d.chars.find(c) != std::string::npos) { out.push_back(cur); cur.clear(); }
        else cur.push_back(c);
    }
    out.push_back(cur);
}
template <class T> T lexical_cast(const std::string &s) { std::istringstream is(s); T v; is >> v; return v; }
template <class T> using shared_ptr = std::shared_ptr<T>;
}  // namespace boost
