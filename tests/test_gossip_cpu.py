"""Gossip membership: several agents in one process on loopback UDP ports (the way the reference tests its membership:
core/src/test/.../GossipTensorParallelMembershipTest)."""
import time

import pytest

from deliverance_b200.parallel.gossip import DeploymentSpec, GossipAgent, TensorParallelMembership


def eventually(fn, timeout=15.0, every=0.05):
    t0 = time.time()
    last = None
    while time.time() - t0 < timeout:
        last = fn()
        if last:
            return last
        time.sleep(every)
    raise AssertionError(f"condition not reached in {timeout} s (last value {last!r})")


class Node:
    def __init__(self, name, seeds, spec, slots=1):
        self.calls = []
        self.agent = GossipAgent(name, ("127.0.0.1", 0), seeds, interval=0.03, fail_after=0.5)
        self.m = TensorParallelMembership(self.agent, spec, slots, "127.0.0.1",
                                          lambda ranks, size, a: self.calls.append(("start", tuple(ranks), size, a.hash)),
                                          lambda: self.calls.append(("stop",)), reconcile_every=0.05)

    def close(self):
        self.m.close()
        self.agent.close()


def cluster(names, spec, slots=None):
    nodes, seeds = [], []
    for n in names:
        node = Node(n, list(seeds), spec, (slots or {}).get(n, 1))
        seeds.append(node.agent.addr)
        nodes.append(node)
    return nodes


def test_election_assignment_and_standby():
    spec = DeploymentSpec("d1", requested_ranks=2, minimum_nodes=3)
    a, b, c = cluster(["a", "b", "c"], spec)
    try:
        eventually(lambda: all(n.m.elected_leader() == "a" for n in (a, b, c)))
        asg = eventually(lambda: c.m.assignment())
        assert asg.ranks == [[0, "a"], [1, "b"]] and asg.size == 2 and asg.leader == "a" and asg.master_port > 0
        topo = c.m.topology()
        assert topo["standby"] == ["c"] and topo["active"] == ["a", "b"]
        eventually(lambda: a.calls and b.calls)
        assert a.calls[0][:3] == ("start", (0,), 2) and b.calls[0][:3] == ("start", (1,), 2) and c.calls == []
        d = b.m.diagnostics()
        assert d["leader"] == "a" and d["local_ranks"] == [1] and d["endpoints"]["a"] == [{"rank": 0, "host": "127.0.0.1"}]
    finally:
        for n in (a, b, c):
            n.close()


def test_standby_takes_over_when_an_active_node_dies():
    spec = DeploymentSpec("d2", requested_ranks=2, minimum_nodes=3)
    a, b, c = cluster(["a", "b", "c"], spec)
    try:
        eventually(lambda: a.calls and b.calls)
        first = a.m.assignment().hash
        b.close()  # the host of rank 1 goes away between steps: its agent stops gossiping
        asg = eventually(lambda: (lambda x: x if x and x.hash != first else None)(a.m.assignment()))
        assert asg.ranks == [[0, "a"], [1, "c"]]
        eventually(lambda: any(call[0] == "start" for call in c.calls))
        assert c.calls[-1][:3] == ("start", (1,), 2)
        # the surviving node restarted its rank for the new group (stop, then start with the new assignment)
        eventually(lambda: [k[0] for k in a.calls].count("start") == 2)
        assert [k[0] for k in a.calls] == ["start", "stop", "start"] and a.calls[-1][3] == asg.hash
    finally:
        for n in (a, c):
            n.close()


def test_new_leader_after_the_leader_dies():
    spec = DeploymentSpec("d3", requested_ranks=2, minimum_nodes=3)
    a, b, c = cluster(["a", "b", "c"], spec)
    try:
        eventually(lambda: b.m.elected_leader() == "a" and b.calls)
        a.close()
        eventually(lambda: b.m.elected_leader() == "b" and c.m.elected_leader() == "b")
        asg = eventually(lambda: (lambda x: x if x and x.leader == "b" else None)(c.m.assignment()))
        assert asg.ranks == [[0, "b"], [1, "c"]]
        eventually(lambda: c.calls and c.calls[-1][:3] == ("start", (1,), 2))
    finally:
        for n in (b, c):
            n.close()


def test_two_slots_on_one_host():
    spec = DeploymentSpec("d4", requested_ranks=2, minimum_nodes=2)
    a, b = cluster(["a", "b"], spec, slots={"a": 2})
    try:
        asg = eventually(lambda: b.m.assignment())
        assert asg.ranks == [[0, "a"], [1, "a"]]
        eventually(lambda: a.calls)
        assert a.calls[0][:3] == ("start", (0, 1), 2) and b.m.topology()["standby"] == ["b"] and b.calls == []
    finally:
        a.close()
        b.close()


def test_manual_assignment():
    spec = DeploymentSpec("d5", requested_ranks=2, minimum_nodes=2, manual=True)
    a, b = cluster(["a", "b"], spec)
    try:
        eventually(lambda: len(a.m.capacities()) == 2)
        time.sleep(0.3)
        assert a.m.assignment() is None and a.calls == []  # nothing happens before ranks are placed
        with pytest.raises(ValueError):
            a.m.assign_rank("a", 2)
        with pytest.raises(ValueError):
            a.m.assign_rank("nobody", 0)
        r = a.m.assign_rank("b", 0)
        assert r["complete"] is False
        with pytest.raises(ValueError):
            a.m.assign_rank("b", 1)  # b offers one slot
        r = a.m.assign_rank("a", 1)
        assert r["complete"] is True
        asg = eventually(lambda: b.m.assignment())
        assert asg.ranks == [[0, "b"], [1, "a"]] and asg.leader == "a"
        eventually(lambda: a.calls and b.calls)
        assert a.calls[0][:3] == ("start", (1,), 2) and b.calls[0][:3] == ("start", (0,), 2)
    finally:
        a.close()
        b.close()


def test_tp_endpoints_serve_the_gossip_view_and_manual_assignment():
    """/tp/gossip and /tp/assign of the HTTP server backed by an observer of a manual-mode deployment."""
    from fastapi.testclient import TestClient

    from deliverance_b200.server.app import ModelRegistry, create_app

    spec = DeploymentSpec("d6", requested_ranks=2, minimum_nodes=2, manual=True)
    a, b = cluster(["a", "b"], spec)
    obs_agent = GossipAgent("server-1", ("127.0.0.1", 0), [a.agent.addr], interval=0.03, fail_after=0.5)
    obs = TensorParallelMembership(obs_agent, spec, candidate=False, reconcile_every=0.05)
    try:
        eventually(lambda: len(obs.capacities()) == 2)
        reg = ModelRegistry()
        reg.membership = obs
        c = TestClient(create_app(reg))
        view = c.get("/tp/gossip").json()
        assert view["membership"] == "gossip" and view["mode"] == "manual" and view["topology"]["active"] == ["a", "b"] and view["assignment"] is None
        assert c.post("/tp/assign", params={"nodeId": "a", "rank": 5}).status_code == 400
        assert c.post("/tp/assign", params={"nodeId": "a", "rank": 0}).json()["complete"] is False
        assert c.post("/tp/assign", params={"nodeId": "b", "rank": 1}).json()["complete"] is True
        eventually(lambda: a.calls and b.calls)
        assert a.calls[0][:3] == ("start", (0,), 2) and b.calls[0][:3] == ("start", (1,), 2)
        assert c.get("/tp/gossip").json()["assignment"]["ranks"] == [[0, "a"], [1, "b"]]
        # without a membership the endpoint keeps its static answer
        assert TestClient(create_app(ModelRegistry())).post("/tp/assign", params={"nodeId": "a", "rank": 0}).status_code == 409
    finally:
        obs.close()
        obs_agent.close()
        a.close()
        b.close()


def test_agents_start_torch_distributed_ranks_from_the_assignment(tmp_path):
    """Two host agents as processes; each starts the rank it is assigned as a child that joins a gloo group at the rendezvous
    address of the assignment and sums over the ranks."""
    import json
    import socket
    import subprocess
    import sys

    s = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    child = ("import os, time, torch, torch.distributed as dist\n"
             "dist.init_process_group('gloo', rank=int(os.environ['RANK']), world_size=int(os.environ['WORLD_SIZE']))\n"
             "t = torch.tensor([float(os.environ['RANK']) + 1.0]); dist.all_reduce(t)\n"
             f"open(os.path.join({str(tmp_path)!r}, 'rank' + os.environ['RANK']), 'w').write(str(t.item()))\n"
             "time.sleep(60)\n")
    base = [sys.executable, "-m", "deliverance_b200.parallel.gossip", "--requested-ranks", "2", "--minimum-nodes", "2", "--deployment", "d7"]
    pa = subprocess.Popen(base + ["--node-id", "a", "--bind", f"127.0.0.1:{port}", "--", sys.executable, "-c", child], stdout=subprocess.PIPE, text=True)
    pb = subprocess.Popen(base + ["--node-id", "b", "--seeds", f"127.0.0.1:{port}", "--", sys.executable, "-c", child], stdout=subprocess.PIPE, text=True)
    try:
        assert json.loads(pa.stdout.readline())["node"] == "a"
        eventually(lambda: (tmp_path / "rank0").exists() and (tmp_path / "rank1").exists() and (tmp_path / "rank0").read_text() != "", timeout=60)
        assert float((tmp_path / "rank0").read_text()) == 3.0 and float((tmp_path / "rank1").read_text()) == 3.0
    finally:
        for p in (pa, pb):
            p.terminate()
        for p in (pa, pb):
            try:
                p.wait(timeout=15)
            except subprocess.TimeoutExpired:
                p.kill()
