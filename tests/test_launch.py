"""Launch tooling: task expansion, script generation, local multi-task run, multi-node rendezvous."""
import os
import subprocess
import sys
import textwrap
import threading

import pytest

EXP_SRC = textwrap.dedent('''
    import os, sys
    from steptronoss_b200.exp.base_exp import BaseExp
    from steptronoss_b200.exp.resources import ResourceConfig, TaskSpec


    class Rsc(ResourceConfig):
        def __init__(self):
            super().__init__()
            self.envs = {"COMMON": "1"}
            self.task_specs = {
                "trainer": TaskSpec(is_critical=True, envs={"ROLE": "trainer"}, command="{PY} {COMMAND}"),
                "helper": TaskSpec(envs={"ROLE": "helper"}, node_type="cpu", replica=REPLICA, command="{PY} {COMMAND}"),
            }


    class Exp(BaseExp):
        resource_cfg = Rsc
        marker = "none"
        log_dir = os.environ.get("OUT_DIR", os.path.dirname(os.path.abspath(__file__)))

        def entrypoint(self):
            self.update_from_args()
            out = os.environ["OUT_DIR"]
            role = os.environ["ROLE"]
            open(os.path.join(out, role + ".txt"), "w").write(f"{self.marker} {os.environ['EXP_ID']} {os.environ['COMMON']}")
            if role == "helper":
                import time
                time.sleep(60)   # must be stopped when the trainer (critical) ends


    if __name__ == "__main__":
        Exp().entrypoint()
''')


def _write_exp(tmp_path, replica=1):
    p = tmp_path / "my_exp.py"
    p.write_text(EXP_SRC.replace("{PY}", sys.executable).replace("REPLICA", str(replica)))
    return str(p)


def test_build_scripts(tmp_path, monkeypatch):
    from steptronoss_b200.launch.build_scripts import build_scripts

    monkeypatch.delenv("EXP_ID", raising=False)
    res = build_scripts(_write_exp(tmp_path, replica=2), str(tmp_path / "out"), ["marker=abc"], exp_id="e1", interactive=False)
    assert len(res.scripts) == 3 and res.exp_id == "e1"
    cpu = sorted(s for s in res.scripts if "/cpu/" in s)
    assert [os.path.basename(s) for s in cpu] == ["0.sh", "1.sh", "2.sh"][: len(cpu)]
    text = open(cpu[-1]).read()
    assert "export EXP_ID=e1/helper" in text and "export ROLE=helper" in text and "export NNODES=2" in text
    assert text.strip().endswith("my_exp.py marker=abc") and os.access(cpu[-1], os.X_OK)


def test_mp_run_stops_helpers_when_critical_task_ends(tmp_path, monkeypatch):
    out = tmp_path / "o"
    out.mkdir()
    env = dict(os.environ, OUT_DIR=str(out), PYTHONPATH=os.getcwd(), EXP_ID="r1")
    r = subprocess.run([sys.executable, "-m", "steptronoss_b200.launch.mp_run", _write_exp(tmp_path), "marker=xyz"],
                       env=env, capture_output=True, text=True, timeout=120, cwd=os.getcwd())
    assert r.returncode == 0, r.stdout + r.stderr
    assert (out / "trainer.txt").read_text() == "xyz r1/trainer 1"
    assert (out / "helper.txt").read_text() == "xyz r1/helper 1"


def test_smartrun_rendezvous_assigns_ranks(tmp_path, monkeypatch):
    from steptronoss_b200.launch.smartrun import rendezvous, torchrun_command
    from steptronoss_b200.utils import comm_utils

    monkeypatch.setenv("STEPTRON_MEET_DIR", str(tmp_path))
    monkeypatch.setenv("EXP_ID", "sr")
    monkeypatch.setenv("SMARTRUN_UNIQUE_PER_PROCESS", "1")
    comm_utils.reset_exp_store()
    store = comm_utils.get_exp_redis()
    # two "nodes": this process and a fake second address pushed by a thread
    t = threading.Timer(0.3, lambda: comm_utils.ExpStore(comm_utils.STORE_ADDR, comm_utils.STORE_PORT)
                        .rpush("SMARTRUN_RDZVS_sr", "10.0.0.2#77"))
    t.start()
    rank, master = rendezvous(2, "sr", poll_s=0.05, store=store)
    assert rank == 0 and master != "10.0.0.2"
    cmd = torchrun_command(["exp.py", "a=1"], 2, rank, master, 12345, 8)
    assert cmd[1:3] == ["-m", "torch.distributed.run"] and cmd[-2:] == ["exp.py", "a=1"] and "--node-rank" in cmd
    comm_utils.reset_exp_store()


def test_submitter_template_resolves_tasks_and_stops_helpers_when_the_critical_task_ends(tmp_path, monkeypatch):
    """A subclass whose ``launch_task`` starts local processes: both tasks get their command, environment and
    rendezvous directory; the helper (which would sleep for a minute) is stopped once the trainer has ended."""
    from steptronoss_b200.launch.example_submitter import Submitter

    monkeypatch.delenv("EXP_ID", raising=False)
    monkeypatch.setenv("OUT_DIR", str(tmp_path))
    seen = {}

    class Local(Submitter):
        poll_s = 0.1
        meet_dir = str(tmp_path / "meet")

        def launch_task(self, sub):
            seen[sub.task.name] = sub
            env = os.environ | sub.task.envs | {"PYTHONPATH": os.getcwd()}
            return subprocess.Popen(sub.task.command, shell=True, env=env)

    with pytest.raises(NotImplementedError):
        Submitter(_write_exp(tmp_path), ["marker=zzz"], interactive=False).run()
    monkeypatch.delenv("EXP_ID", raising=False)
    subs = Local(_write_exp(tmp_path), ["marker=zzz"], image="img:1", interactive=False).run()
    assert set(seen) == {"trainer", "helper"}
    t, h = seen["trainer"], seen["helper"]
    assert t.task.is_critical and not h.task.is_critical and t.image == "img:1"
    assert t.task.envs["ROLE"] == "trainer" and t.task.envs["COMMON"] == "1" and t.task.envs["NNODES"] == "1"
    exp_id = t.task.envs["EXP_ID"].split("/")[0]
    assert t.task.envs["EXP_ID"] == f"{exp_id}/trainer" and h.task.envs["EXP_ID"] == f"{exp_id}/helper"
    assert t.task.envs["STEPTRON_MEET_DIR"] == os.path.join(str(tmp_path / "meet"), exp_id, "trainer")
    assert "marker=zzz" in t.task.command
    assert open(tmp_path / "trainer.txt").read().split()[0] == "zzz"
    for s in subs:
        s.handle.wait(timeout=10)
        assert s.handle.poll() is not None
