/* Test infrastructure (not part of the product): exhaustive check of the encoder's element-type
 * quotient (packkv_b200/csrc/quant_dev.cuh, HalfQuotient) against the reference's arithmetic.
 *
 * The reference quantiser computes round(x / scale) on fp16 / bf16 tensors (utils/compute.py:97-104):
 * PyTorch divides in fp32 and rounds to the element type, then rounds half to even.  The GPU path
 * instead evaluates r = RN(1/scale), q0 = RN(x*r), e = RN(fma(-pre*scale, q0, pre*x)),
 * q1 = RN(fma(e, r/pre, q0)) in the element type (pre = 128 for fp16, 1 for bf16) and rounds q1 half
 * to even.  This program restates both in double precision with explicit round-to-nearest-even to the
 * element type and compares the resulting integers for every scale whose biased exponent lies in
 * [lo, hi] and every x >= 0 with |x / scale| <= 512 for which pre*x is finite (the kernels check both
 * conditions and otherwise use the fp32 path).  Signs are symmetric.
 *
 *   half_quotient_check <bf16: 0|1> <lo exponent> <hi exponent> <pre>      prints "... bad N of M ..."
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

static int MB, EMIN, EMAX, BIAS; /* explicit mantissa bits, minimum normal exponent, maximum exponent, bias */

static double decode(uint16_t h) {
    const int emax = (1 << (15 - MB)) - 1;
    const int s = h >> 15, e = (h >> MB) & emax, m = h & ((1 << MB) - 1);
    double v;
    if (e == 0) v = ldexp((double)m, EMIN - MB);
    else if (e == emax) v = m ? NAN : INFINITY;
    else v = ldexp((double)(m | (1 << MB)), e - BIAS - MB);
    return s ? -v : v;
}

/* round an exactly known double to the element type, ties to even, gradual underflow */
static double rn(double x) {
    if (x == 0 || isnan(x) || isinf(x)) return x;
    int e;
    const double a = fabs(x);
    frexp(a, &e);
    int lsb = e - 1 - MB;
    if (lsb < EMIN - MB) lsb = EMIN - MB;
    double r = ldexp(nearbyint(ldexp(a, -lsb)), lsb);
    if (r > ldexp(2.0 - ldexp(1.0, -MB), EMAX)) r = INFINITY;
    return x < 0 ? -r : r;
}

int main(int argc, char** argv) {
    if (argc < 5) return 2;
    const int bf = atoi(argv[1]), lo_e = atoi(argv[2]), hi_e = atoi(argv[3]);
    const double pre = atof(argv[4]);
    if (bf) { MB = 7; EMIN = -126; EMAX = 127; BIAS = 127; } else { MB = 10; EMIN = -14; EMAX = 15; BIAS = 15; }
    long bad = 0, total = 0, skipped_scales = 0;
    for (int sb = lo_e << MB; sb < ((hi_e + 1) << MB); sb++) {
        const double s = decode((uint16_t)sb);
        if (!(s > 0) || isinf(s)) continue;
        const double r = rn((double)(float)(1.0 / s));             /* __float2half_rn(__frcp_rn(scale)) */
        const double sp = rn(s * pre), rp = rn(r / pre);
        if (sp != s * pre || rp != r / pre) { skipped_scales++; continue; }   /* scalings must be exact */
        for (int xb = 0; xb < 0x8000; xb++) {
            const double x = decode((uint16_t)xb);
            if (isnan(x) || isinf(x)) continue;
            const double ref = rn((double)((float)x / (float)s));  /* the reference: fp32 division, then the element type */
            if (!(fabs(ref) <= 512.0)) continue;
            const double xp = rn(x * pre);
            if (xp != x * pre) continue;
            const double q0 = rn(x * r);
            const double e = rn(fma(-sp, q0, xp));
            const double q1 = rn(fma(e, rp, q0));
            total++;
            if (nearbyint(q1) != nearbyint(ref)) {
                if (bad++ < 8) printf("scale %04x x %04x: %.10g vs %.10g\n", sb, xb, q1, ref);
            }
        }
    }
    printf("bf16=%d exponents %d..%d pre=%g: bad %ld of %ld (scales skipped: %ld)\n", bf, lo_e, hi_e, pre, bad, total, skipped_scales);
    return bad != 0;
}
