"""The decode kernel's alternative paths, each forced by its environment switch in a child process (the switches
are read once per process): the merge through global scratch instead of a cluster, the cluster merge that meets
at a cluster barrier instead of completing the receiver's mbarrier, launches without programmatic dependent
launch, the driver's default cluster placement, bulk copies forced on for selection lists and off for dense
scans, the reference's split-count knob, and the two-level merge of long scans instead of the merge by all of the
unit's blocks.  Every child runs the same parity tests against the oracle."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = ["test_gpu_decode.py::test_config1_ctx4096_reference_check",
         "test_gpu_decode.py::test_qsa_sparse_decode_per_kv_head_lists",
         "test_gpu_decode.py::test_batched_sessions_match_single_session",
         "test_gpu_decode.py::test_sequence_shards_partial_and_merge",
         "test_gpu_fused_append.py"]


@pytest.mark.parametrize("switch", ["Q4_DEC_CLUSTER=0", "Q4_DEC_PUSH_ASYNC=0", "Q4_DEC_PDL=0", "Q4_DEC_CLUSTER_POLICY=0",
                                    "Q4_DEC_BULK=1", "Q4_DEC_BULK=0", "Q4_DEC_SPLIT_S=5", "Q4_DEC_GRIDMERGE=0"])
def test_parity_with_the_switch_set(switch):
    env = dict(os.environ)
    name, value = switch.split("=")
    env[name] = value
    cmd = [sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu", "-p", "no:cacheprovider"] + [os.path.join(HERE, c) for c in CASES]
    r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=900)
    assert r.returncode == 0, "%s:\n%s" % (switch, r.stdout[-3000:])
