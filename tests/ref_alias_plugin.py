"""pytest plugin (``-p ref_alias_plugin``) for running the reference's own tests against this library.

The reference's test helper only looks at backends named "cuda", "triton" and "eager"
(``tests/conftest.py:70-90`` of the reference), and its compiled "cuda" backend does not exist on the GPU box, so this
plugin registers this library's operators under the name "cuda" as well as under their own name "sm100", in front of
the others, before any reference test module is imported.  ``tests/test_gpu_registry.py`` starts pytest with it in a
child process on the copy of the reference tests that ``baseline/make_ref.py`` makes; nothing else uses it.
"""
from __future__ import annotations

import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    ref = os.path.join(ROOT, "baseline", "_ref")
    for p in (ref, ROOT):
        if p not in sys.path:
            sys.path.insert(0, p)
    import comfy_kitchen_b200 as ckb
    from comfy_kitchen.registry import registry
    ckb.install()                            # "sm100", first in priority
    ckb.install(name="cuda", first=False)    # the name the reference's helper looks for
    registry.set_priority(["sm100", "cuda", "triton", "eager"])
    import comfy_kitchen as ck
    info = ck.list_backends()
    assert info["cuda"]["available"] and "scaled_mm_nvfp4" in info["cuda"]["capabilities"]
    config._ckb_launches_at_start = ckb.launches()


def pytest_terminal_summary(terminalreporter, exitstatus, config):
    import comfy_kitchen_b200 as ckb
    import torch
    n = ckb.launches() - getattr(config, "_ckb_launches_at_start", 0)
    status = ckb.read_device_status() if torch.cuda.is_available() else -1
    terminalreporter.write_line(f"CKB_KERNEL_LAUNCHES={n} CKB_DEVICE_STATUS={status}")
