"""The reference-side binding include/tensorlib_b200_device.hpp (class B200 : CUDA<half>).

CPU: it must compile against the reference's own headers (every `override` has to match a virtual of
Device<half>, tensorLib/include/device/Device.hpp:13-98) and link with the reference's objects and
the product library. Needs the reference checkout (TL_REFERENCE_ROOT, default the place the oracle
Makefile uses); skipped where it is absent.
GPU: the prebuilt check program calls every virtual on the reference's CUDA<half> object and on a
B200 object over the same device data and compares (tests/cpp/shim_check.cpp)."""
import os
import subprocess

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
CHECK = os.path.join(ROOT, "oracle", "_ref", "shim_check")


def test_binding_compiles_and_links_against_the_reference():
    ref_root = os.environ.get("TL_REFERENCE_ROOT", "/root/reference")
    if not os.path.isdir(os.path.join(ref_root, "tensorLib", "include")):
        pytest.skip("reference checkout not present")
    if not os.path.exists(os.path.join(ROOT, "tensorlib_b200", "libtensorlib_b200.so")):
        subprocess.run(["python", "-m", "tensorlib_b200.build"], cwd=ROOT, check=True)
    r = subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), f"REF={ref_root}", "ref", "ref_shim", "-j8"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    r = subprocess.run([CHECK, "--link-only"], capture_output=True, text=True)
    assert r.returncode == 0 and "linked" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_every_device_virtual_agrees_between_the_reference_cuda_object_and_the_binding():
    if not os.path.exists(CHECK):
        pytest.skip("oracle/_ref/shim_check not built (needs the reference checkout at build time)")
    r = subprocess.run([CHECK], capture_output=True, text=True, timeout=300)
    print(r.stdout)
    assert r.returncode == 0 and "SHIM OK" in r.stdout, r.stdout[-4000:] + r.stderr[-2000:]
