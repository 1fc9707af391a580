"""The quantize kernels replace `x / d` by a reciprocal plus one fused correction step
(tensorrt_b200/csrc/exact_div.h).  This compiles that header as C and checks it against
IEEE division on tens of millions of operand pairs, including the structured operands the
kernels see (bf16 / fp16 numerators, E4M3-times-fp32 divisors)."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent

SRC = r"""
#include <stdio.h>
#include <stdlib.h>
#include "exact_div.h"
static uint64_t s = 88172645463325252ULL;
static inline uint64_t rng(void){ s ^= s<<13; s ^= s>>7; s ^= s<<17; return s; }
static inline float bits(uint32_t u){ float f; memcpy(&f,&u,4); return f; }
int main(int argc, char** argv){
  long n = atol(argv[1]); long bad = 0;
  for (int mode = 0; mode < 4; ++mode) for (long i = 0; i < n; ++i) {
    uint32_t ra = (uint32_t)rng(), rb = (uint32_t)rng();
    uint32_t ea = 90 + (ra >> 23) % 76, eb = 90 + (rb >> 23) % 76;
    uint32_t ma = ra & 0x7fffff, mb = rb & 0x7fffff;
    if (mode == 1) ma &= 0x7f0000;            /* bf16 numerator */
    if (mode == 2) ma &= 0x7fe000;            /* fp16 numerator */
    float a = bits((ea << 23) | ma), d = bits((eb << 23) | mb);
    if (mode == 3) {                           /* divisor = e4m3 value * fp32 global scale */
      float e4 = (float)(8 + (rb & 7)) * 0.125f;  /* 1.xxx with 3 mantissa bits */
      d = e4 * d;
      ma &= 0x7f0000; a = bits((ea << 23) | ma);
    }
    if (!b200q_div_fast_ok(d)) continue;
    if (ra & 0x80000000u) a = -a;              /* both signs */
    if ((i & 0xfffff) == 0) a = (i & 0x100000) ? -0.0f : 0.0f;   /* signed zeros */
    float y = b200q_rcp_rn(d);
    float q = b200q_div_by_shared(a, d, y);
    if (b200q_f32_bits(q) != b200q_f32_bits(a / d)) { if (bad < 5) printf("mismatch a=%a d=%a got=%a want=%a\n", a, d, q, a / d); ++bad; }
  }
  printf("bad=%ld\n", bad);
  return bad != 0;
}
"""


@pytest.mark.skipif(shutil.which("gcc") is None, reason="gcc not available")
def test_shared_divisor_sequence_equals_ieee_division(tmp_path):
    src = tmp_path / "divcheck.c"
    src.write_text(SRC)
    exe = tmp_path / "divcheck"
    subprocess.run(["gcc", "-O2", "-mfma", "-ffp-contract=off", "-I", str(ROOT / "tensorrt_b200" / "csrc"),
                    str(src), "-o", str(exe), "-lm"], check=True)
    out = subprocess.run([str(exe), "10000000"], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout
    assert "bad=0" in out.stdout
