// Postfix expression builder over the REFERENCE's public Expression API, shared by the dumpers in this folder.
//
// TEST AND BASELINE INFRASTRUCTURE ONLY (never shipped, never linked by the product).  Nothing of the reference is
// copied here: the builder only calls Expression's public methods (Utilities/Expression/Expression.h:516-1075).
//
// Program: tokens separated by blanks.  in:<name>  rs:<name> (fp32 runtime scalar)  lit:<value>  cast:<dtype int>
// binary: add sub mul div pow min max   unary: the names below   reductions: rsum / rmean / rmax / rmin / rprod / rnorm1 /
// rnorm2 followed by :<axes> and optionally :<squeeze axes> (comma separated, e.g. rmean:1 or rsum:0,1:0).
#pragma once

#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "Utilities/Expression/Expression.h"

namespace thor_ref_dump {

using ThorImplementation::DataType;
using ThorImplementation::Expression;

inline Expression unaryByName(const Expression& x, const std::string& op) {
#define TB_U(NAME) if (op == #NAME) return x.NAME();
    TB_U(abs) TB_U(ceil) TB_U(floor) TB_U(round) TB_U(trunc) TB_U(sin) TB_U(cos) TB_U(tan) TB_U(asin) TB_U(acos) TB_U(atan) TB_U(sinh) TB_U(cosh)
    TB_U(asinh) TB_U(acosh) TB_U(atanh) TB_U(erf) TB_U(erfc) TB_U(erfcx) TB_U(erfinv) TB_U(erfcinv) TB_U(tgamma) TB_U(lgamma) TB_U(digamma) TB_U(ln)
    TB_U(log1p) TB_U(log2) TB_U(log10) TB_U(exp) TB_U(expm1) TB_U(exp2) TB_U(exp10) TB_U(sqrt) TB_U(normcdf) TB_U(sigmoid) TB_U(tanh) TB_U(softplus)
    TB_U(selu) TB_U(gelu) TB_U(relu6) TB_U(swish)
#undef TB_U
    if (op == "neg") return -x;
    if (op == "relu") return x.max(Expression(0.0));
    throw std::invalid_argument("unknown unary op '" + op + "'");
}

inline std::vector<uint64_t> axisList(const std::string& text) {
    std::vector<uint64_t> out;
    std::istringstream is(text);
    std::string item;
    while (std::getline(is, item, ','))
        if (!item.empty()) out.push_back(std::stoull(item));
    return out;
}

inline Expression buildFromPostfix(const std::string& program) {
    std::vector<Expression> stack;
    std::istringstream is(program);
    std::string tok;
    auto pop = [&]() {
        if (stack.empty()) throw std::invalid_argument("postfix program pops an empty stack");
        Expression e = stack.back();
        stack.pop_back();
        return e;
    };
    while (is >> tok) {
        if (tok.rfind("in:", 0) == 0) stack.push_back(Expression::input(tok.substr(3)));
        else if (tok.rfind("rs:", 0) == 0) stack.push_back(Expression::runtimeScalar(tok.substr(3)));
        else if (tok.rfind("lit:", 0) == 0) stack.push_back(Expression(std::stod(tok.substr(4))));
        else if (tok.rfind("cast:", 0) == 0) {
            Expression a = pop();
            stack.push_back(a.cast(static_cast<DataType>(std::stoi(tok.substr(5)))));
        } else if (tok.size() > 1 && tok[0] == 'r' && tok.find(':') != std::string::npos && tok.rfind("rs:", 0) != 0) {
            const size_t c1 = tok.find(':'), c2 = tok.find(':', c1 + 1);
            const std::string name = tok.substr(0, c1);
            const std::vector<uint64_t> axes = axisList(tok.substr(c1 + 1, c2 == std::string::npos ? std::string::npos : c2 - c1 - 1));
            const std::vector<uint64_t> squeeze = c2 == std::string::npos ? std::vector<uint64_t>{} : axisList(tok.substr(c2 + 1));
            Expression a = pop();
            if (name == "rsum") stack.push_back(a.reduce_sum(axes, squeeze));
            else if (name == "rmean") stack.push_back(a.reduce_mean(axes, squeeze));
            else if (name == "rmax") stack.push_back(a.reduce_max(axes, squeeze));
            else if (name == "rmin") stack.push_back(a.reduce_min(axes, squeeze));
            else if (name == "rprod") stack.push_back(a.reduce_prod(axes, squeeze));
            else if (name == "rnorm1") stack.push_back(a.reduce_norm1(axes, squeeze));
            else if (name == "rnorm2") stack.push_back(a.reduce_norm2(axes, squeeze));
            else throw std::invalid_argument("unknown reduction '" + name + "'");
        } else if (tok == "add" || tok == "sub" || tok == "mul" || tok == "div" || tok == "pow" || tok == "min" || tok == "max") {
            Expression b = pop();
            Expression a = pop();
            stack.push_back(tok == "add" ? a + b : tok == "sub" ? a - b : tok == "mul" ? a * b : tok == "div" ? a / b : tok == "pow" ? a.pow(b)
                            : tok == "min" ? a.min(b) : a.max(b));
        } else {
            Expression a = pop();
            stack.push_back(unaryByName(a, tok));
        }
    }
    if (stack.size() != 1) throw std::invalid_argument("postfix program must leave exactly one value");
    return stack.back();
}

}  // namespace thor_ref_dump
