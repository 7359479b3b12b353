"""The control plane: registry with expiry and scopes, the engine-side client (heartbeat, re-registration after the registry forgot
the entry), and the C++ gateway discovering and dropping engines through it."""
import json
import os
import socket
import subprocess
import threading
import time
import urllib.request

import pytest

from nanoengine_b200.server.ctrl import CtrlClient, Registry, advertise_host, make_server

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GATEWAY = os.path.join(ROOT, "nanoengine_b200", "_native", "ne-gateway")


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _serve(ttl=15.0):
    port = _port()
    srv = make_server("127.0.0.1", port, ttl)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    return srv, f"http://127.0.0.1:{port}"


def test_registry_expiry_scopes_and_validation():
    t = [0.0]
    reg = Registry(ttl=10.0, clock=lambda: t[0])
    reg.register({"id": "a", "host": "h1", "port": 8000, "role": "prefill", "model": "m", "scope": "blue"})
    reg.register({"id": "b", "port": 8001, "model": "m"})
    assert {e["id"] for e in reg.list()} == {"a", "b"} and [e["id"] for e in reg.list("blue")] == ["a"]
    assert reg.list("blue")[0]["url"] == "http://h1:8000" and reg.list()[1]["role"] == "hybrid"
    t[0] = 8.0
    assert reg.heartbeat("a") and not reg.heartbeat("nobody")
    t[0] = 12.0                                   # b was last seen at 0: gone; a at 8: alive
    assert [e["id"] for e in reg.list()] == ["a"]
    t[0] = 30.0
    assert not reg.heartbeat("a") and reg.list() == []
    with pytest.raises(ValueError):
        reg.register({"id": "x", "port": 1, "role": "router"})
    with pytest.raises(ValueError):
        reg.register({"host": "h"})
    assert advertise_host("10.1.2.3") == "10.1.2.3" and advertise_host("0.0.0.0")


def test_client_registers_heartbeats_and_comes_back_after_being_forgotten():
    srv, url = _serve()
    try:
        cli = CtrlClient(url, scope="blue")
        assert cli.register("e0", "127.0.0.1", 8000, role="decode", model="m", engine_id="d0")
        ents = cli.list_entities()
        assert len(ents) == 1 and ents[0]["role"] == "decode" and ents[0]["scope"] == "blue" and ents[0]["engine_id"] == "d0"
        assert CtrlClient(url, scope="green").list_entities() == []
        cli.start_heartbeat(interval=0.05)
        srv.registry.unregister("e0")              # the registry lost the entry (a restart)
        for _ in range(100):
            if cli.list_entities():
                break
            time.sleep(0.02)
        assert [e["id"] for e in cli.list_entities()] == ["e0"]
        cli.stop()
        assert cli.list_entities() == []
        assert not CtrlClient("http://127.0.0.1:1", timeout=0.2).register("x", "h", 1)      # nobody listening: False, no exception
        assert json.loads(urllib.request.urlopen(url + "/health").read())["status"] == "ok"
    finally:
        srv.shutdown()


@pytest.mark.skipif(not os.path.exists(GATEWAY), reason="gateway binary not built")
def test_gateway_discovers_engines_through_the_control_plane():
    from test_gateway import FakeEngine, _post
    srv, url = _serve(ttl=1.5)
    e = FakeEngine("hybrid")
    port = _port()
    gw = subprocess.Popen([GATEWAY, "--port", str(port), "--host", "127.0.0.1", "--ctrl-address", url], stderr=subprocess.DEVNULL)
    cli = CtrlClient(url)
    try:
        assert cli.register("e0", "127.0.0.1", e.port, model="m")
        cli.start_heartbeat(interval=0.1)
        base = f"http://127.0.0.1:{port}"
        for _ in range(100):
            try:
                if json.loads(urllib.request.urlopen(base + "/status").read())["engines"]["hybrid"]:
                    break
            except OSError:
                pass
            time.sleep(0.1)
        assert _post(base + "/v1/completions", {"prompt": "x"})[0] == 200
        cli._stop.set()                             # the engine falls silent (no unregister): its entry expires, the gateway drops it
        for _ in range(120):
            if not json.loads(urllib.request.urlopen(base + "/status").read())["engines"]["hybrid"]:
                break
            time.sleep(0.1)
        assert _post(base + "/v1/completions", {"prompt": "x"})[0] == 503
    finally:
        gw.terminate(); e.stop(); srv.shutdown()


def test_engine_registration_carries_role_model_scope_and_engine_id():
    from nanoengine_b200 import Config
    from nanoengine_b200.server.ctrl import register_with_ctrl
    srv, url = _serve()
    try:
        cfg = Config(model="tiny-deepseek-v3", device="cpu", dtype="float32", mode="prefill", engine_id="p7", ctrl_address=url, ctrl_scope="blue",
                     served_model_name="tiny")
        cli = register_with_ctrl(cfg, "127.0.0.1", 8123, cfg.served_model_name)
        assert cli is not None
        (ent,) = CtrlClient(url, scope="blue").list_entities()
        assert ent["role"] == "prefill" and ent["model"] == "tiny" and ent["engine_id"] == "p7" and ent["url"] == "http://127.0.0.1:8123"
        cli.stop()
        assert CtrlClient(url).list_entities() == []
        assert register_with_ctrl(Config(model="tiny-deepseek-v3", device="cpu", dtype="float32", ctrl_address="http://127.0.0.1:1"), "127.0.0.1", 1, "m") is None
    finally:
        srv.shutdown()


def test_engine_component_publishes_its_description_and_peers_read_it_back():
    """`LLMComponent` registers the engine's own description (what a peer checks before it accepts migrated sequences) and keeps it
    alive; after the registry forgot it, the next heartbeat brings it back."""
    from nanoengine_b200 import Config, LLMComponent
    srv, url = _serve()
    comp = None
    try:
        comp = LLMComponent(Config(model="tiny-deepseek-v3", device="cpu", dtype="float32", kvcache_block_size=16, num_kvcache_blocks=16,
                                   max_num_seqs=2, engine_id="d3", mode="decode", ctrl_address=url))
        assert comp.registered
        req = urllib.request.Request(url + "/get_entity", json.dumps({"id": "d3"}).encode(), {"Content-Type": "application/json"})
        ent = json.loads(urllib.request.urlopen(req).read())["entity"]
        assert ent["id"] == "d3" and ent["block_size"] == 16 and ent == comp.engine_info()
        srv.registry.unregister("d3")
        for _ in range(100):
            if srv.registry.get_engine("d3") is not None:
                break
            time.sleep(0.1)
        assert srv.registry.get_engine("d3") is not None
        assert CtrlClient(url).list_entities() == []              # an engine description is not an HTTP endpoint: gateways do not see it
    finally:
        if comp is not None:
            comp.shutdown()
        srv.shutdown()


def test_decode_engine_finds_its_prefill_peer_through_the_control_plane():
    """No `pd_peers`: the first sequence migrated from an unknown prefill engine makes the decode engine look that engine up in the
    control plane and connect to the endpoint its description names (the connector is substituted: CPU engines share memory, GPU
    engines would map each other's pools).  The tokens equal the hybrid engine's; an engine the control plane does not know is asked
    for once."""
    import torch
    from nanoengine_b200 import Config, LLM, RequestMigrate, SamplingParams
    from nanoengine_b200.parallel.kv_transfer import KVMigrator, LocalTransport
    from nanoengine_b200.server.ctrl import EnginePublisher
    srv, url = _serve()
    pub = None
    try:
        base = dict(model="tiny-deepseek-v3", dtype="float32", device="cpu", kvcache_block_size=16, max_num_seqs=8, num_kvcache_blocks=64)
        g = torch.Generator().manual_seed(21)
        prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (30, 17)]
        sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
        want = {o["seq_id"]: o["token_ids"] for o in LLM(Config(**base)).generate(prompts, sp)}
        prefill = LLM(Config(**base, mode="prefill", engine_id="p0", engine_endpoint="ipc:///tmp/ne-test-p0.sock"))
        decode = LLM(Config(**base, mode="decode", engine_id="d0", ctrl_address=url))
        pub = EnginePublisher(url, prefill.engine.engine_info, interval=0.2)
        assert pub.published
        calls = []

        def connect(engine, eid, endpoint):
            calls.append((eid, endpoint))
            tr = LocalTransport([prefill.engine.executor.runner], [engine.executor.runner])
            engine.migrator = KVMigrator(tr, engine.engine_info(), prefill.engine.engine_info())

        decode.engine._pd_connect = connect
        firsts = {}
        for b in prefill.generate(prompts, sp, return_serialized=True):
            sid, first = RequestMigrate.from_bytes(b).metadata
            firsts[sid] = first
            decode.add_request_payload(b)
        outs = {o["seq_id"]: [firsts[o["seq_id"]]] + o["token_ids"] for o in decode.generate()}
        assert outs == want and calls == [("p0", "ipc:///tmp/ne-test-p0.sock")]            # looked up and connected once
        # a sequence from an engine nobody published
        lone = LLM(Config(**base, mode="prefill", engine_id="ghost"))
        blob = lone.generate(prompts[:1], sp, return_serialized=True)[0]
        decode.add_request_payload(blob)
        decode.generate()               # takes the migrator's default route; the lookup is made once and remembered as failed
        assert "ghost" in decode.engine._pd_unresolved and len(calls) == 1
    finally:
        if pub is not None:
            pub.stop()
        srv.shutdown()


def test_ctrl_command_line_and_config_flags():
    import sys
    from nanoengine_b200.server.cli import parse_config_args
    port = _port()
    p = subprocess.Popen([sys.executable, "-m", "nanoengine_b200.server.cli", "ctrl", "--host", "127.0.0.1", "--port", str(port), "--ttl", "3"],
                         cwd=ROOT, stderr=subprocess.DEVNULL)
    try:
        url = f"http://127.0.0.1:{port}"
        for _ in range(100):
            try:
                if json.loads(urllib.request.urlopen(url + "/health", timeout=0.5).read())["status"] == "ok":
                    break
            except OSError:
                time.sleep(0.1)
        cli = CtrlClient(url)
        assert cli.register("e0", "127.0.0.1", 8000, model="m") and len(cli.list_entities()) == 1
    finally:
        p.terminate()
        p.wait(timeout=10)
    common, roles = parse_config_args(["--ctrl_address", "http://h:4479", "--ctrl-scope", "blue", "--served_model_name", "m", "--engine_endpoint",
                                       "ipc:///tmp/x.sock", "--pd_peers", '{"p0": "ipc:///tmp/p0.sock"}', "--status_log_interval_s", "0",
                                       "--fp8_scale_format", "ue8m0", "--decode.max_num_seqs", "64"])
    assert common["ctrl_scope"] == "blue" and common["pd_peers"] == {"p0": "ipc:///tmp/p0.sock"} and common["status_log_interval_s"] == 0.0
    assert common["fp8_scale_format"] == "ue8m0" and common["engine_endpoint"] == "ipc:///tmp/x.sock" and roles["decode"] == {"max_num_seqs": 64}
