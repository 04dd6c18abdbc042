"""Every device buffer between guard bands (GB200_CANARIES=1): training with all three optimizers and decoding with all
three token-step forms on sizes that do not divide the tile shapes must leave the bands untouched."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_no_kernel_writes_outside_its_buffers(tmp_path):
    env = dict(os.environ, GB200_CANARIES="1")
    p = subprocess.run([sys.executable, os.path.join(os.path.dirname(__file__), "canary_worker.py"), str(tmp_path)],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env, timeout=900)
    assert p.returncode == 0 and "CANARIES OK" in p.stdout, p.stdout[-3000:]


def test_the_guard_check_sees_a_stray_write(monkeypatch):
    import torch
    from ghassan_b200.utils import canary as CA
    monkeypatch.setenv("GB200_CANARIES", "1")
    CA.reset()
    t = CA.zeros(5, 7, dtype=torch.float16, device="cuda", name="probe")
    assert t.shape == (5, 7) and t.data_ptr() % 256 == 0 and CA.check() == []
    flat = t.view(-1)
    torch.as_strided(flat, (1,), (1,), storage_offset=flat.storage_offset() + 35).fill_(1.0)   # one element past the end
    assert CA.check() == ["probe:above"]
    CA.reset()
    monkeypatch.delenv("GB200_CANARIES")
    assert CA.zeros(4, dtype=torch.float32, device="cuda").numel() == 4 and CA.count() == 0
