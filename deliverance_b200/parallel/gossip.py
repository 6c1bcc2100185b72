"""Gossip membership for tensor-parallel deployments: liveness, capacity, leader election, rank assignment, reconcile.

What the reference does with its UDP gossip library (core/.../model/tensorparallel/GossipParallelMembership.java:36-689): every
node publishes how many ranks it can host (capacity), the live nodes sorted by id fill the requested ranks in order and the rest
are standby (topology, :197-218), every active node votes for the first active node and the leader is the candidate that has the
votes of all active nodes (majority-vote CRDT, :244-258, :418-434), the leader publishes the assignment rank -> node (:436-458)
and a rendezvous address, and every node runs a reconcile loop (every 500 ms) that stops and restarts its local ranks whenever
the ranks assigned to it or the group size change (:368-416). A manual mode takes rank assignments one by one
(``POST /tp/assign``, :460-533) and publishes the assignment once all ranks are placed.

Here the transport is a small UDP gossip of JSON state between the nodes' agents (one agent per host, not per GPU):

* per-node state (heartbeat counter, capacity, rank endpoints) travels with a version per key; the copy with the higher version
  wins; a node whose heartbeat has not advanced for ``fail_after`` seconds is down;
* shared state is a map of last-writer-wins registers ordered by (Lamport clock, writer id), plus the vote map
  candidate -> {voter: active view}, merged by union with the later vote of a voter winning.

The ranks themselves are ordinary ``torch.distributed`` processes: the worker callback gets ``(ranks, world_size, assignment)``
and starts one process per local rank with ``RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT`` taken from the assignment (the
leader's host and the published rendezvous port); ``python -m deliverance_b200.parallel.gossip ... -- <command>`` does that with
:mod:`subprocess`. Everything here runs on the host; tests run several agents in one process on loopback ports.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import random
import signal
import socket
import subprocess
import sys
import threading
import time
from dataclasses import dataclass
from typing import Callable, Optional


@dataclass
class DeploymentSpec:
    """What is to be deployed (the reference's ``deliverance.tp.*`` keys, TensorParallelDeploymentSpec.java:9-58)."""
    deployment_id: str = "default"
    requested_ranks: int = 2
    minimum_nodes: int = 1
    manual: bool = False


@dataclass
class Assignment:
    deployment_id: str
    leader: str
    size: int
    hash: str
    ranks: list  # [[rank, node_id], ...]
    master_port: int = 0
    leader_host: str = "127.0.0.1"

    def ranks_for(self, node_id: str) -> list:
        return [int(r) for r, n in self.ranks if n == node_id]


def assignment_hash(deployment_id: str, slots: int, active: list) -> str:
    return hashlib.sha256(json.dumps([deployment_id, slots, active]).encode()).hexdigest()[:16]


class GossipAgent:
    """UDP gossip of per-node and shared state between a handful of hosts."""

    def __init__(self, node_id: str, bind=("127.0.0.1", 0), seeds=(), interval: float = 0.1, fail_after: float = 1.5, fanout: int = 3):
        self.node_id, self.interval, self.fail_after, self.fanout = node_id, interval, fail_after, fanout
        self.sock = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
        self.sock.bind(tuple(bind))
        self.sock.settimeout(0.05)
        self.addr = self.sock.getsockname()
        self.seeds = [tuple(s) for s in seeds]
        self.lock = threading.RLock()
        self.clock = 0
        # node_id -> {"addr": [host, port], "hb": int, "data": {key: [version, value]}}
        self.nodes = {node_id: {"addr": list(self.addr), "hb": 0, "data": {}}}
        self.seen = {node_id: time.monotonic()}
        self.shared: dict = {}   # key -> [clock, writer, value]
        self.votes: dict = {}    # vote key -> {candidate: {voter: [clock, active_view]}}
        self.closed = False
        self.listeners: list = []
        self.threads = [threading.Thread(target=self._recv_loop, daemon=True), threading.Thread(target=self._send_loop, daemon=True)]
        for t in self.threads:
            t.start()

    # ------------------------------------------------------------------ local writes
    def set_node_data(self, key: str, value) -> None:
        with self.lock:
            cur = self.nodes[self.node_id]["data"].get(key, [0, None])
            self.nodes[self.node_id]["data"][key] = [cur[0] + 1, value]

    def put_shared(self, key: str, value) -> None:
        with self.lock:
            self.clock += 1
            self.shared[key] = [self.clock, self.node_id, value]

    def vote(self, key: str, candidate: str, active_view: list) -> None:
        with self.lock:
            self.clock += 1
            self.votes.setdefault(key, {}).setdefault(candidate, {})[self.node_id] = [self.clock, list(active_view)]

    # ------------------------------------------------------------------ reads
    def live_nodes(self) -> list:
        now = time.monotonic()
        with self.lock:
            return sorted(n for n in self.nodes if n == self.node_id or now - self.seen.get(n, 0.0) <= self.fail_after)

    def node_data(self, node_id: str, key: str):
        with self.lock:
            ent = self.nodes.get(node_id, {}).get("data", {}).get(key)
            return None if ent is None else ent[1]

    def get_shared(self, key: str):
        with self.lock:
            ent = self.shared.get(key)
            return None if ent is None else ent[2]

    def get_votes(self, key: str) -> dict:
        with self.lock:
            return {c: {v: list(e[1]) for v, e in vs.items()} for c, vs in self.votes.get(key, {}).items()}

    def snapshot(self) -> dict:
        with self.lock:
            return {"node": self.node_id, "addr": list(self.addr), "live": self.live_nodes(), "known": sorted(self.nodes),
                    "shared_keys": sorted(self.shared), "clock": self.clock}

    # ------------------------------------------------------------------ wire
    def _state(self) -> bytes:
        with self.lock:
            self.nodes[self.node_id]["hb"] += 1
            live = set(self.live_nodes())
            nodes = {n: e for n, e in self.nodes.items() if n in live}  # the dead are not spread further
            return json.dumps({"from": self.node_id, "clock": self.clock, "nodes": nodes, "shared": self.shared, "votes": self.votes}).encode()

    def _merge(self, msg: dict) -> None:
        now = time.monotonic()
        with self.lock:
            self.clock = max(self.clock, int(msg.get("clock", 0)))
            for n, ent in msg.get("nodes", {}).items():
                if n == self.node_id:
                    continue
                cur = self.nodes.get(n)
                if cur is None:
                    self.nodes[n] = {"addr": ent["addr"], "hb": ent["hb"], "data": dict(ent.get("data", {}))}
                    self.seen[n] = now
                    continue
                if ent["hb"] > cur["hb"]:
                    cur["hb"], cur["addr"] = ent["hb"], ent["addr"]
                    self.seen[n] = now
                for k, (ver, val) in ent.get("data", {}).items():
                    if ver > cur["data"].get(k, [0, None])[0]:
                        cur["data"][k] = [ver, val]
            for k, (clk, writer, val) in msg.get("shared", {}).items():
                cur = self.shared.get(k)
                if cur is None or (clk, writer) > (cur[0], cur[1]):
                    self.shared[k] = [clk, writer, val]
            for k, cands in msg.get("votes", {}).items():
                mine = self.votes.setdefault(k, {})
                for cand, voters in cands.items():
                    dst = mine.setdefault(cand, {})
                    for voter, (clk, view) in voters.items():
                        if voter not in dst or clk > dst[voter][0]:
                            dst[voter] = [clk, view]
        for fn in list(self.listeners):
            fn()

    def _recv_loop(self) -> None:
        while not self.closed:
            try:
                data, _ = self.sock.recvfrom(1 << 16)
            except socket.timeout:
                continue
            except OSError:
                return
            try:
                self._merge(json.loads(data.decode()))
            except (ValueError, KeyError, TypeError):
                continue  # a malformed datagram is dropped

    def _send_loop(self) -> None:
        rng = random.Random(hash(self.node_id) & 0xFFFF)
        while not self.closed:
            payload = self._state()
            with self.lock:
                peers = [tuple(e["addr"]) for n, e in self.nodes.items() if n != self.node_id and n in self.live_nodes()]
            targets = set(rng.sample(peers, min(self.fanout, len(peers)))) | set(self.seeds)
            targets.discard(tuple(self.addr))
            for t in targets:
                try:
                    self.sock.sendto(payload, t)
                except OSError:
                    pass
            time.sleep(self.interval)

    def close(self) -> None:
        self.closed = True
        try:
            self.sock.close()
        except OSError:
            pass


class TensorParallelMembership:
    """Capacity, topology, election, assignment and the reconcile loop on top of a :class:`GossipAgent`."""

    def __init__(self, agent: GossipAgent, spec: DeploymentSpec, slots: int = 1, host: str = "127.0.0.1",
                 start_ranks: Optional[Callable] = None, stop_ranks: Optional[Callable] = None, candidate: bool = True,
                 reconcile_every: float = 0.5):
        self.agent, self.spec, self.slots, self.host, self.candidate = agent, spec, slots, host, candidate
        self.start_ranks, self.stop_ranks = start_ranks, stop_ranks
        self.reconcile_every = reconcile_every
        self.k_cap = f"tp/{spec.deployment_id}/capacity"
        self.k_vote = f"tp/{spec.deployment_id}/leader"
        self.k_assign = f"tp/{spec.deployment_id}/assignment"
        self.k_manual = f"tp/{spec.deployment_id}/manual"
        self.k_endpoints = f"tp/{spec.deployment_id}/endpoints"
        self.running_ranks: list = []
        self.running_size = 0
        self.running_hash = ""
        self.events: list = []
        self.closed = False
        self.formed = False
        if candidate:
            agent.set_node_data(self.k_cap, {"slots": int(slots), "host": host})
        self.thread = threading.Thread(target=self._coordinate, daemon=True)
        self.thread.start()

    # ------------------------------------------------------------------ views
    def capacities(self) -> list:
        out = []
        for n in self.agent.live_nodes():
            cap = self.agent.node_data(n, self.k_cap)
            if cap:
                out.append((n, int(cap["slots"]), cap.get("host", "127.0.0.1")))
        return out

    def topology(self) -> dict:
        """Live nodes in id order fill the requested ranks with their slots; nodes that are not needed are standby."""
        active, standby, slots = [], [], 0
        for n, s, _ in self.capacities():
            slots += s
            if len(active) < self.spec.requested_ranks:
                active += [n] * min(s, self.spec.requested_ranks - len(active))
            else:
                standby.append(n)
        return {"deployment": self.spec.deployment_id, "slots": slots, "rank_nodes": active, "active": sorted(set(active)),
                "standby": standby, "hash": assignment_hash(self.spec.deployment_id, slots, active)}

    def elected_leader(self) -> Optional[str]:
        if self.spec.manual:
            a = self.assignment()
            return a.leader if a else None
        active = self.topology()["active"]
        if not active:
            return None
        for cand, voters in self.agent.get_votes(self.k_vote).items():
            if cand in active and all(v in voters and sorted(voters[v]) == active for v in active):
                return cand
        return None

    def assignment(self) -> Optional[Assignment]:
        raw = self.agent.get_shared(self.k_assign)
        return Assignment(**raw) if raw else None

    def diagnostics(self) -> dict:
        a = self.assignment()
        return {"node": self.agent.node_id, "deployment": self.spec.deployment_id, "mode": "manual" if self.spec.manual else "election",
                "live": self.agent.live_nodes(), "topology": self.topology(), "leader": self.elected_leader(),
                "assignment": a.__dict__ if a else None, "local_ranks": list(self.running_ranks), "events": self.events[-20:],
                "endpoints": {n: self.agent.node_data(n, self.k_endpoints) for n in self.agent.live_nodes()}}

    # ------------------------------------------------------------------ election and assignment
    def vote_if_needed(self) -> None:
        topo = self.topology()
        if self.agent.node_id in topo["active"] and self.elected_leader() is None:
            self.agent.vote(self.k_vote, topo["active"][0], topo["active"])

    def publish_assignment_as_leader(self) -> bool:
        topo = self.topology()
        if self.elected_leader() != self.agent.node_id or len(topo["rank_nodes"]) < self.spec.requested_ranks:
            return False
        cur = self.assignment()
        if cur is not None and cur.hash == topo["hash"] and cur.leader == self.agent.node_id:
            return True
        port = _free_port()
        hosts = {n: h for n, _, h in self.capacities()}
        a = Assignment(self.spec.deployment_id, self.agent.node_id, len(topo["rank_nodes"]), topo["hash"],
                       [[r, n] for r, n in enumerate(topo["rank_nodes"])], port, hosts.get(topo["rank_nodes"][0], self.host))  # rendezvous where rank 0 runs
        self.agent.put_shared(self.k_assign, a.__dict__)
        self.events.append(f"published assignment {a.hash} ranks={a.ranks}")
        return True

    def assign_rank(self, node_id: str, rank: int) -> dict:
        """Manual mode: place one rank; the assignment is published once every rank has a node (reference :460-533)."""
        if not self.spec.manual:
            raise RuntimeError("manual rank assignment needs a deployment in manual mode")
        if rank < 0 or rank >= self.spec.requested_ranks:
            raise ValueError(f"rank must be between 0 and {self.spec.requested_ranks - 1}")
        caps = {n: s for n, s, _ in self.capacities()}
        if node_id not in caps:
            raise ValueError(f"no live capacity for node {node_id}")
        draft = dict(self.agent.get_shared(self.k_manual) or {})
        draft[str(rank)] = node_id
        per_node: dict = {}
        for n in draft.values():
            per_node[n] = per_node.get(n, 0) + 1
            if n not in caps:
                raise ValueError(f"no live capacity for node {n}")
            if per_node[n] > caps[n]:
                raise ValueError(f"node {n} would get {per_node[n]} ranks, capacity {caps[n]}")
        self.agent.put_shared(self.k_manual, draft)
        if len(draft) == self.spec.requested_ranks:
            nodes = [draft[str(r)] for r in range(self.spec.requested_ranks)]
            hosts = {n: h for n, _, h in self.capacities()}
            a = Assignment(self.spec.deployment_id, self.agent.node_id, len(nodes), assignment_hash(self.spec.deployment_id, sum(caps.values()), nodes),
                           [[r, n] for r, n in enumerate(nodes)], _free_port(), hosts.get(nodes[0], self.host))
            self.agent.put_shared(self.k_assign, a.__dict__)
            self.events.append(f"published manual assignment ranks={a.ranks}")
        return {"deployment": self.spec.deployment_id, "ranks": draft, "complete": len(draft) == self.spec.requested_ranks}

    def publish_endpoints(self, endpoints: list) -> None:
        self.agent.set_node_data(self.k_endpoints, endpoints)

    # ------------------------------------------------------------------ reconcile loop
    def _reconcile(self) -> None:
        a = self.assignment()
        live = set(self.agent.live_nodes())
        if a is not None and not self.spec.manual and any(n not in live for _, n in a.ranks):
            a_valid = False  # a node of the assignment is down: its ranks are gone, wait for the leader's new assignment
        else:
            a_valid = a is not None
        want = a.ranks_for(self.agent.node_id) if a_valid else []
        size = a.size if a_valid else 0
        h = a.hash if a_valid else ""
        if want == self.running_ranks and size == self.running_size and h == self.running_hash:
            return
        if self.running_ranks:
            self.events.append(f"stopping ranks {self.running_ranks}")
            if self.stop_ranks:
                self.stop_ranks()
            self.publish_endpoints([])
        self.running_ranks, self.running_size, self.running_hash = list(want), size, h
        if want:
            self.events.append(f"starting ranks {want} of {size} ({h})")
            if self.start_ranks:
                self.start_ranks(list(want), size, a)
            self.publish_endpoints([{"rank": r, "host": self.host} for r in want])

    def _coordinate(self) -> None:
        while not self.closed:
            try:
                # the minimum number of hosts gates only the first election (voting on an incomplete view would place ranks on
                # the early arrivals); afterwards the group shrinks and grows with the live hosts
                if not self.spec.manual and not self.formed and len(self.capacities()) >= self.spec.minimum_nodes:
                    self.formed = True
                if not self.spec.manual and self.formed:
                    self.vote_if_needed()
                    if self.elected_leader() == self.agent.node_id:
                        self.publish_assignment_as_leader()
                if self.candidate:
                    self._reconcile()
            except Exception as e:  # noqa: BLE001 - the loop must survive a callback's failure
                self.events.append(f"coordination error: {e!r}")
            time.sleep(min(self.reconcile_every, 0.1) if not self.running_ranks else self.reconcile_every)

    def close(self) -> None:
        self.closed = True
        if self.running_ranks and self.stop_ranks:
            self.stop_ranks()
        self.running_ranks = []


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class ProcessRanks:
    """Worker callbacks that run one child process per local rank with the torch.distributed environment of the assignment."""

    def __init__(self, command: list, gpus_from: int = 0, extra_env: Optional[dict] = None):
        self.command, self.gpus_from, self.procs, self.extra_env = command, gpus_from, [], dict(extra_env or {})

    def start(self, ranks: list, size: int, a: Assignment) -> None:
        for i, r in enumerate(ranks):
            env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(size), LOCAL_RANK=str(self.gpus_from + i), MASTER_ADDR=a.leader_host,
                       MASTER_PORT=str(a.master_port), DLV_TP_ASSIGNMENT=a.hash, **self.extra_env)
            self.procs.append(subprocess.Popen(self.command, env=env))

    def stop(self) -> None:
        for p in self.procs:
            if p.poll() is None:
                p.terminate()
        for p in self.procs:
            try:
                p.wait(timeout=10)
            except subprocess.TimeoutExpired:
                p.kill()
        self.procs = []


def observer_from_env(node_id: str) -> Optional[TensorParallelMembership]:
    """A non-candidate member built from ``DLV_GOSSIP_SEEDS`` / ``DLV_TP_*`` (set by the host's agent for its rank processes): it
    follows the gossip, offers no capacity and starts no ranks. ``None`` when the process is not gossip-managed."""
    seeds = os.environ.get("DLV_GOSSIP_SEEDS", "")
    if not seeds:
        return None
    pairs = [(s.rsplit(":", 1)[0], int(s.rsplit(":", 1)[1])) for s in seeds.split(",") if s]
    spec = DeploymentSpec(os.environ.get("DLV_TP_DEPLOYMENT", "default"), int(os.environ.get("DLV_TP_REQUESTED_RANKS", "2")), 1,
                          os.environ.get("DLV_TP_MANUAL", "0") == "1")
    agent = GossipAgent(node_id, ("127.0.0.1", 0), pairs)
    return TensorParallelMembership(agent, spec, candidate=False)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="gossip agent of one host: joins the deployment and runs the ranks it is assigned")
    ap.add_argument("--node-id", required=True)
    ap.add_argument("--bind", default="127.0.0.1:0")
    ap.add_argument("--seeds", default="", help="comma list of host:port of other agents")
    ap.add_argument("--deployment", default="default")
    ap.add_argument("--requested-ranks", type=int, default=2)
    ap.add_argument("--minimum-nodes", type=int, default=1)
    ap.add_argument("--slots", type=int, default=1, help="ranks (GPUs) this host offers")
    ap.add_argument("--host", default="127.0.0.1", help="address other hosts reach this one at")
    ap.add_argument("--manual", action="store_true")
    ap.add_argument("command", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    cmd = a.command[1:] if a.command[:1] == ["--"] else a.command
    host, port = a.bind.rsplit(":", 1)
    seeds = [(s.rsplit(":", 1)[0], int(s.rsplit(":", 1)[1])) for s in a.seeds.split(",") if s]
    agent = GossipAgent(a.node_id, (host, int(port)), seeds)
    # the rank processes can watch the deployment as observers (the HTTP server of rank 0 serves /tp/gossip and /tp/assign from it)
    child_env = {"DLV_GOSSIP_SEEDS": f"{agent.addr[0]}:{agent.addr[1]}", "DLV_TP_DEPLOYMENT": a.deployment,
                 "DLV_TP_REQUESTED_RANKS": str(a.requested_ranks), "DLV_TP_MANUAL": "1" if a.manual else "0"}
    ranks = ProcessRanks(cmd, extra_env=child_env) if cmd else None
    m = TensorParallelMembership(agent, DeploymentSpec(a.deployment, a.requested_ranks, a.minimum_nodes, a.manual), a.slots, a.host,
                                 ranks.start if ranks else None, ranks.stop if ranks else None)
    print(json.dumps({"node": a.node_id, "gossip": list(agent.addr)}), flush=True)

    def _terminate(*_):  # SIGTERM ends the agent the way Ctrl-C does: the local ranks are stopped first
        raise KeyboardInterrupt

    signal.signal(signal.SIGTERM, _terminate)
    try:
        while True:
            time.sleep(5)
            print(json.dumps(m.diagnostics()), flush=True)
    except KeyboardInterrupt:
        pass
    finally:
        m.close()
        agent.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
