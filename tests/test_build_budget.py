"""Compile-time budget of the whole-token decode kernel (no GPU needed).

The kernel runs 17 warps per SM, so ptxas may use at most 96 registers per thread; it sits close to that limit, and
one more live value in the wrong place moves the projection loop's state to local memory (measured: a 720-byte stack
frame made the gate/up phase 5x slower).  This test reads ptxas' own report and fails when the frame grows."""
import os
import re
import subprocess

from ironmill_b200 import build


def test_decode_token_kernel_keeps_its_state_in_registers(tmp_path):
    src = os.path.join(build.CSRC, "decode_mega.cu")
    cmd = [build._nvcc(), *build.NVCC_FLAGS, "-Xptxas", "-v", "-I", build.INCLUDE, "-c", src, "-o", str(tmp_path / "m.o")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    frames = {}
    name = None
    for line in r.stderr.splitlines():
        m = re.search(r"Function properties for (\S+)", line)
        if m:
            name = m.group(1)
        m = re.search(r"(\d+) bytes stack frame", line)
        if m and name and "decode_token_kernel" in name:
            frames[name] = int(m.group(1))
    assert len(frames) == 12, frames         # GQ = 1, 2, 4, 8: single-GPU and tensor-parallel for the 8-bit cache, single-GPU for the 4-bit one
    # single-GPU instantiations (Lb0E) and tensor-parallel ones (Lb1E: the mailbox reads cost a few more live values)
    assert max(f for n, f in frames.items() if "Lb0E" in n) <= 160, frames
    assert max(f for n, f in frames.items() if "Lb1E" in n) <= 224, frames
