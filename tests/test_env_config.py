"""Configuration variables of the reference that this library honours on the host side: a user-supplied topology
file, escalation to INFO after the first warning, and the variables that select transports (accepted, reported)."""
from tests.mp_util import run_ranks


def _worker(lib, uid, rank, world):
    comm = lib.flagcxCommInitRank(world, uid, rank)
    lib.flagcxCommDestroy(comm)
    return True


def test_topology_file_is_read_and_checked(native_lib, tmp_path):
    topo = tmp_path / "topo.xml"
    topo.write_text('<system version="1" domain="nvswitch" ranks="2" multicast="0">\n  <gpu dev="0" net="mlx5_0"></gpu>\n'
                    '  <gpu dev="1" net="mlx5_1"></gpu>\n</system>\n')
    log = tmp_path / "log_%p.txt"
    env = {"FLAGCX_TOPO_FILE": str(topo), "FLAGCX_DEBUG": "INFO", "FLAGCX_DEBUG_SUBSYS": "GRAPH,ENV", "FLAGCX_DEBUG_FILE": str(log),
           "FLAGCX_USE_HETERO_COMM": "1", "CUDA_VISIBLE_DEVICES": ""}
    run_ranks(_worker, 2, env=env)
    text = "".join(p.read_text() for p in tmp_path.glob("log_*.txt"))
    assert "network port known for 2 of 2 ranks" in text
    assert "FLAGCX_USE_HETERO_COMM=1 accepted" in text


def test_topology_file_with_wrong_world_warns_and_escalates(native_lib, tmp_path):
    topo = tmp_path / "topo.xml"
    topo.write_text('<system version="1" domain="nvswitch" ranks="8" multicast="1">\n</system>\n')
    log = tmp_path / "log_%p.txt"
    env = {"FLAGCX_TOPO_FILE": str(topo), "FLAGCX_DEBUG": "WARN", "FLAGCX_WARN_ENABLE_DEBUG_INFO": "1", "FLAGCX_DEBUG_FILE": str(log),
           "CUDA_VISIBLE_DEVICES": ""}
    run_ranks(_worker, 2, env=env)
    text = "".join(p.read_text() for p in tmp_path.glob("log_*.txt"))
    assert "describes 8 ranks, the communicator has 2" in text
    assert "FLAGCX INFO" in text  # INFO lines appear only because the warning switched them on
