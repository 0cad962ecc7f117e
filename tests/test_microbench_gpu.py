"""The per-kernel timing script runs each of its three modes (small shapes) and prints one line per launch."""
import pytest

from denograd_b200 import microbench

pytestmark = pytest.mark.gpu


def test_every_mode_prints_its_lines(capsys):
    small = ["--dim", "512", "--hidden", "1024", "--heads", "8", "--kv-heads", "2", "--repeat", "2"]
    microbench.main(["projections", "--rows", "160"] + small)
    microbench.main(["prefill-attention", "--positions", "100", "--start", "30", "--batch", "2"] + small)
    microbench.main(["decode-attention", "--batch", "9", "--context", "300"] + small)
    out = capsys.readouterr().out.splitlines()
    assert len(out) == 7 and all(" us " in line for line in out), out
    assert out[4].split()[2] == "layer"
