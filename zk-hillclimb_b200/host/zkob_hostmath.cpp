// The host-side field arithmetic of the driver programs (zkob_common.hpp: BLS12-381 scalar field add / sub / mul / inverse, the
// signed-integer lift, the Lagrange evaluations of the round polynomials, the one-variable eq factor) behind a line protocol, so
// that it can be checked against exact integer arithmetic without a GPU.  One request per stdin line:
//   <op> <hex> <hex> ...      op in add sub mul inv i64 lag3 lag4 lag5 eq1;  numbers as big-endian hex (i64: a signed decimal)
// and one big-endian hex answer per line.  Nothing here touches the device.
#include "zkob_common.hpp"

#include <sstream>

using namespace zkob;

namespace {

Fr from_hex(const std::string& h) {
    Fr r{};
    int nib = 0;
    for (size_t i = h.size(); i-- > 0 && nib < 64; nib++) {
        const char ch = h[i];
        const uint32_t v = ch >= '0' && ch <= '9' ? ch - '0' : ch >= 'a' && ch <= 'f' ? ch - 'a' + 10 : ch >= 'A' && ch <= 'F' ? ch - 'A' + 10 : 0;
        r.v[nib / 8] |= v << (4 * (nib % 8));
    }
    return r;
}
std::string to_hex(const Fr& a) {
    char buf[72];
    for (int i = 0; i < 8; i++) snprintf(buf + 8 * i, 9, "%08x", a.v[7 - i]);
    return buf;
}

}  // namespace

int main() {
    std::string line;
    while (std::getline(std::cin, line)) {
        std::istringstream in(line);
        std::string op, tok;
        in >> op;
        std::vector<std::string> a;
        while (in >> tok) a.push_back(tok);
        std::vector<Fr> f;
        if (op != "i64") for (const std::string& s : a) f.push_back(from_hex(s));
        Fr r{};
        const Fr inv2 = fr_inv(fr_u32(2)), inv4 = fr_inv(fr_u32(4)), inv6 = fr_inv(fr_u32(6)), inv24 = fr_inv(fr_u32(24));
        if (op == "add" && f.size() == 2) r = fr_add(f[0], f[1]);
        else if (op == "sub" && f.size() == 2) r = fr_sub(f[0], f[1]);
        else if (op == "mul" && f.size() == 2) r = fr_mul(f[0], f[1]);
        else if (op == "inv" && f.size() == 1) r = fr_inv(f[0]);
        else if (op == "i64" && a.size() == 1) r = fr_from_i64(strtoll(a[0].c_str(), nullptr, 10));
        else if (op == "lag3" && f.size() == 4) r = lagrange3(f[0], f[1], f[2], f[3]);
        else if (op == "lag4" && f.size() == 5) r = lagrange4({f[0], f[1], f[2], f[3]}, f[4], inv6, inv2);
        else if (op == "lag5" && f.size() == 6) r = lagrange5({f[0], f[1], f[2], f[3], f[4]}, f[5], inv24, inv6, inv4);
        else if (op == "eq1" && f.size() == 2) r = eq1(f[0], f[1]);
        else { std::cout << "?" << std::endl; continue; }
        std::cout << to_hex(r) << std::endl;
    }
    return 0;
}
