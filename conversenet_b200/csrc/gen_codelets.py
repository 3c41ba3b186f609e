#!/usr/bin/env python3
"""Generate `fft_codelets.cuh`: straight-line, register-resident DFT butterflies.

Each codelet `Radix<R>::fwd(re, im)` computes the un-normalised forward DFT
(kernel exp(-2*pi*i*n*k/R)) of R complex values held in two register arrays,
natural order in, natural order out.  The inverse is the same routine with the
real and imaginary arrays swapped.

Construction
  * R = 2, 4      : the usual add/sub butterflies.
  * R odd prime   : the conjugate-pair form.  With s_j = x_j + x_{R-j} and
                    d_j = x_j - x_{R-j},  a_k = x_0 + sum_j cos(2 pi jk/R) s_j,
                    b_k = sum_j sin(2 pi jk/R) d_j,  X_k = a_k - i b_k,
                    X_{R-k} = a_k + i b_k.  About R fused multiply-adds per point.
  * R composite   : one Cooley-Tukey split A x B with literal twiddles, the
                    sub-transforms generated recursively.

Usage:  python gen_codelets.py > fft_codelets.cuh   (the build does this).
"""
import math
import sys

RADICES = [2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 22, 23, 24, 26]


def is_prime(n):
    return n > 1 and all(n % d for d in range(2, int(n ** 0.5) + 1))


def flit(v):
    if v == 0:
        return "0.0f"
    return repr(float(v)) + "f"


class Emitter:
    def __init__(self):
        self.lines = []
        self.n = 0

    def tmp(self):
        self.n += 1
        return f"t{self.n}"

    def let(self, expr):
        name = self.tmp()
        self.lines.append(f"    const float {name} = {expr};")
        return name

    def add(self, a, b):
        return self.let(f"{a} + {b}")

    def sub(self, a, b):
        return self.let(f"{a} - {b}")

    def neg(self, a):
        return self.let(f"-{a}")

    # complex helpers on (re, im) name pairs
    def cadd(self, x, y):
        return (self.add(x[0], y[0]), self.add(x[1], y[1]))

    def csub(self, x, y):
        return (self.sub(x[0], y[0]), self.sub(x[1], y[1]))

    def mul_neg_i(self, x):  # (a+ib)(-i) = b - ia
        return (x[1], self.neg(x[0]))

    def twiddle(self, x, num, den):
        """x * exp(-2 pi i num/den)."""
        num %= den
        if num == 0:
            return x
        if 4 * num == den:
            return self.mul_neg_i(x)
        if 2 * num == den:
            return (self.neg(x[0]), self.neg(x[1]))
        if 4 * num == 3 * den:  # * (+i): (a+ib) i = -b + ia
            return (self.neg(x[1]), x[0])
        th = 2.0 * math.pi * num / den
        c, s = math.cos(th), math.sin(th)
        if 8 * num % den == 0:  # odd multiples of 1/8 turn: |c| == |s|
            r = math.sqrt(0.5)
            # (a+ib)(c - is) with c = sc*r, s = ss*r
            sc = 1.0 if c > 0 else -1.0
            ss = 1.0 if s > 0 else -1.0
            # re = r*(sc*a + ss*b), im = r*(sc*b - ss*a)
            ra = x[0] if sc > 0 else f"(-{x[0]})"
            rb = x[1] if sc > 0 else f"(-{x[1]})"
            re = self.let(f"{flit(r)} * ({ra} {'+' if ss > 0 else '-'} {x[1]})")
            im = self.let(f"{flit(r)} * ({rb} {'-' if ss > 0 else '+'} {x[0]})")
            return (re, im)
        # re = a c + b s ; im = b c - a s
        re = self.let(f"fmaf({x[1]}, {flit(s)}, {x[0]} * {flit(c)})")
        im = self.let(f"fmaf({x[1]}, {flit(c)}, -({x[0]} * {flit(s)}))")
        return (re, im)

    def dft(self, xs):
        R = len(xs)
        if R == 1:
            return list(xs)
        if R == 2:
            return [self.cadd(xs[0], xs[1]), self.csub(xs[0], xs[1])]
        if R == 4:
            a = self.cadd(xs[0], xs[2])
            b = self.csub(xs[0], xs[2])
            c = self.cadd(xs[1], xs[3])
            d = self.mul_neg_i(self.csub(xs[1], xs[3]))
            return [self.cadd(a, c), self.cadd(b, d), self.csub(a, c), self.csub(b, d)]
        if is_prime(R):
            return self.dft_odd_prime(xs)
        if R % 4 == 0:
            A = 4
        elif R % 2 == 0:
            A = 2
        else:
            A = next(d for d in range(3, R) if R % d == 0)
        B = R // A
        u = [None] * R
        for j in range(B):
            t = self.dft([xs[j + B * q] for q in range(A)])
            for p in range(A):
                u[p * B + j] = self.twiddle(t[p], j * p, R)
        out = [None] * R
        for p in range(A):
            z = self.dft([u[p * B + j] for j in range(B)])
            for p1 in range(B):
                out[p + A * p1] = z[p1]
        return out

    def dft_odd_prime(self, xs):
        R = len(xs)
        hn = (R - 1) // 2
        s = [None] + [self.cadd(xs[j], xs[R - j]) for j in range(1, hn + 1)]
        d = [None] + [self.csub(xs[j], xs[R - j]) for j in range(1, hn + 1)]
        # X_0
        accr, acci = xs[0]
        for j in range(1, hn + 1):
            accr = self.add(accr, s[j][0])
            acci = self.add(acci, s[j][1])
        out = [None] * R
        out[0] = (accr, acci)
        for k in range(1, hn + 1):
            ar, ai = xs[0]
            br = bi = None
            for j in range(1, hn + 1):
                th = 2.0 * math.pi * ((j * k) % R) / R
                c, sn = math.cos(th), math.sin(th)
                ar = self.let(f"fmaf({flit(c)}, {s[j][0]}, {ar})")
                ai = self.let(f"fmaf({flit(c)}, {s[j][1]}, {ai})")
                if br is None:
                    br = self.let(f"{flit(sn)} * {d[j][0]}")
                    bi = self.let(f"{flit(sn)} * {d[j][1]}")
                else:
                    br = self.let(f"fmaf({flit(sn)}, {d[j][0]}, {br})")
                    bi = self.let(f"fmaf({flit(sn)}, {d[j][1]}, {bi})")
            out[k] = (self.add(ar, bi), self.sub(ai, br))
            out[R - k] = (self.sub(ar, bi), self.add(ai, br))
        return out


class Emitter2(Emitter):
    """The same butterflies on PACKED complex values: one 64-bit register pair holds (re, im) and the
    additions, multiplications by a real constant and fused multiply-adds act on both halves with one
    instruction (add / mul / fma .f32x2 of sm_100).  Nearly every operation of these codelets treats the
    real and the imaginary part alike, so the instruction count of a butterfly drops by about 40 %.
    A value name stands for a `p2` variable."""

    def let(self, expr):
        name = self.tmp()
        self.lines.append(f"    const p2 {name} = {expr};")
        return name

    @staticmethod
    def both(v):
        return f"p2_pack({flit(v)}, {flit(v)})"

    def cadd(self, x, y):
        return self.let(f"p2_add({x}, {y})")

    def csub(self, x, y):
        return self.let(f"p2_sub({x}, {y})")

    def parts(self, x):
        r, i = self.tmp(), self.tmp()
        self.lines.append(f"    float {r}, {i}; p2_unpack({x}, {r}, {i});")
        return r, i

    def mul_neg_i(self, x):  # (a+ib)(-i) = b - ia
        r, i = self.parts(x)
        return self.let(f"p2_pack({i}, -{r})")

    def mul_pos_i(self, x):  # (a+ib) i = -b + ia
        r, i = self.parts(x)
        return self.let(f"p2_pack(-{i}, {r})")

    def twiddle(self, x, num, den):
        """x * exp(-2 pi i num/den)."""
        num %= den
        if num == 0:
            return x
        if 4 * num == den:
            return self.mul_neg_i(x)
        if 2 * num == den:
            return self.let(f"p2_mul({x}, {self.both(-1.0)})")
        if 4 * num == 3 * den:
            return self.mul_pos_i(x)
        th = 2.0 * math.pi * num / den
        c, s = math.cos(th), math.sin(th)
        # (a + ib)(c - is) = (a c + b s, b c - a s) = (a, b) * (c, c) + (b, a) * (s, -s)
        r, i = self.parts(x)
        sw = self.let(f"p2_pack({i}, {r})")
        return self.let(f"p2_fma({sw}, p2_pack({flit(s)}, {flit(-s)}), p2_mul({x}, {self.both(c)}))")

    def dft_odd_prime(self, xs):
        R = len(xs)
        hn = (R - 1) // 2
        s = [None] + [self.cadd(xs[j], xs[R - j]) for j in range(1, hn + 1)]
        d = [None] + [self.csub(xs[j], xs[R - j]) for j in range(1, hn + 1)]
        acc = xs[0]
        for j in range(1, hn + 1):
            acc = self.cadd(acc, s[j])
        out = [None] * R
        out[0] = acc
        for k in range(1, hn + 1):
            a = xs[0]
            b = None
            for j in range(1, hn + 1):
                th = 2.0 * math.pi * ((j * k) % R) / R
                c, sn = math.cos(th), math.sin(th)
                a = self.let(f"p2_fma({self.both(c)}, {s[j]}, {a})")
                if b is None:
                    b = self.let(f"p2_mul({self.both(sn)}, {d[j]})")
                else:
                    b = self.let(f"p2_fma({self.both(sn)}, {d[j]}, {b})")
            # X_k = a - i b = a + (b.im, -b.re),  X_{R-k} = a + i b = a - (b.im, -b.re)
            w = self.mul_neg_i(b)
            out[k] = self.cadd(a, w)
            out[R - k] = self.csub(a, w)
        return out


def gen(R):
    e = Emitter()
    xs = [(f"re[{i}]", f"im[{i}]") for i in range(R)]
    out = e.dft(xs)
    e2 = Emitter2()
    out2 = e2.dft([f"z{i}" for i in range(R)])
    lines = [f"template <> struct Radix<{R}> {{",
             f"  static CVB_HD void fwd(float (&re)[{R}], float (&im)[{R}]) {{",
             "#if defined(__CUDA_ARCH__) && !defined(CVB_SCALAR_CODELETS)"]
    for i in range(R):
        lines.append(f"    const p2 z{i} = p2_pack(re[{i}], im[{i}]);")
    lines += e2.lines
    for i, z in enumerate(out2):
        lines.append(f"    p2_unpack({z}, re[{i}], im[{i}]);")
    lines.append("#else")
    lines += e.lines
    for i, (r, m) in enumerate(out):
        lines.append(f"    const float o{i}r = {r}, o{i}i = {m};")
    for i in range(R):
        lines.append(f"    re[{i}] = o{i}r; im[{i}] = o{i}i;")
    lines += ["#endif", "  }", "};", ""]
    return "\n".join(lines)


def main():
    print("// GENERATED by gen_codelets.py -- do not edit.  Register-resident DFT butterflies.")
    print("#pragma once")
    print("#ifndef CVB_HD")
    print("#define CVB_HD __host__ __device__ __forceinline__")
    print("#endif")
    print("namespace cvb {")
    print("#ifdef __CUDA_ARCH__")
    print("// packed (re, im) pairs and the two-wide fp32 instructions of sm_100")
    print("typedef unsigned long long p2;")
    print("__device__ __forceinline__ p2 p2_pack(float x, float y) { p2 r; asm(\"mov.b64 %0, {%1, %2};\" : \"=l\"(r) : \"f\"(x), \"f\"(y)); return r; }")
    print("__device__ __forceinline__ void p2_unpack(p2 v, float& x, float& y) { asm(\"mov.b64 {%0, %1}, %2;\" : \"=f\"(x), \"=f\"(y) : \"l\"(v)); }")
    print("__device__ __forceinline__ p2 p2_add(p2 a, p2 b) { p2 r; asm(\"add.rn.f32x2 %0, %1, %2;\" : \"=l\"(r) : \"l\"(a), \"l\"(b)); return r; }")
    print("__device__ __forceinline__ p2 p2_sub(p2 a, p2 b) { p2 r; asm(\"sub.rn.f32x2 %0, %1, %2;\" : \"=l\"(r) : \"l\"(a), \"l\"(b)); return r; }")
    print("__device__ __forceinline__ p2 p2_mul(p2 a, p2 b) { p2 r; asm(\"mul.rn.f32x2 %0, %1, %2;\" : \"=l\"(r) : \"l\"(a), \"l\"(b)); return r; }")
    print("__device__ __forceinline__ p2 p2_fma(p2 a, p2 b, p2 c) { p2 r; asm(\"fma.rn.f32x2 %0, %1, %2, %3;\" : \"=l\"(r) : \"l\"(a), \"l\"(b), \"l\"(c)); return r; }")
    print("#endif")
    print("template <int R> struct Radix;")
    print("template <> struct Radix<1> { static CVB_HD void fwd(float (&)[1], float (&)[1]) {} };")
    print()
    for R in RADICES:
        print(gen(R))
    print("#define CVB_FOR_EACH_RADIX(X) " + " ".join(f"X({R})" for R in RADICES))
    print("static const int kRadices[] = {" + ", ".join(str(R) for R in RADICES) + "};")
    print("static const int kNumRadices = %d;" % len(RADICES))
    print("}  // namespace cvb")


if __name__ == "__main__":
    main()
