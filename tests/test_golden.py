"""The host layer and the oracle against fixtures recorded from the reference itself
(tests/golden/make_golden.py)."""
import json
import os
import random

import pytest

from bikv_b200 import taskinfo as pb
from bikv_b200.page_manager import MultiPageManager, PageManager
from bikv_b200.plan import build_plan
from oracle import bikv_oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    with open(os.path.join(GOLD, name)) as f:
        return json.load(f)


def _run(fn, *a):
    try:
        return fn(*a)
    except Exception as e:  # noqa: BLE001
        return type(e).__name__


@pytest.mark.parametrize("trace", [t for t in load("page_manager.json") if t["kind"] == "single"],
                         ids=lambda t: f"{t['cache_size']}x{t['page_size']}")
def test_page_manager_matches_reference_trace(trace):
    pm = PageManager(trace["cache_size"], trace["page_size"])
    for op, iid, ln, want in trace["ops"]:
        if op == "load":
            got = _run(pm.load_item, iid, ln)
            got = got if isinstance(got, str) else [list(got[0]), list(got[1])]
        elif op == "access":
            got = _run(pm.access_item, iid)
            got = got if isinstance(got, str) else list(got)
        elif op == "protect":
            got = _run(pm.set_protected, iid)
        else:
            got = _run(pm.remove_protected, iid)
        assert got == want, (op, iid, ln)
    assert pm.get_loaded_lists() == trace["loaded"]
    assert list(pm.free_pages) == trace["free"]


@pytest.mark.parametrize("trace", [t for t in load("page_manager.json") if t["kind"] == "multi"],
                         ids=lambda t: f"{t['cache_size']}x{t['page_size']}x{t['shards']}")
def test_multi_page_manager_matches_reference_trace(trace):
    random.seed(trace["random_seed"])
    mpm = MultiPageManager(trace["cache_size"], trace["page_size"], trace["shards"])
    for op, iid, ln, want in trace["ops"]:
        if op == "load":
            got = _run(mpm.load_item, iid, ln)
            got = got if isinstance(got, str) else [got[0], list(got[1])]
        else:
            s, pages = mpm.access_item(iid)
            got = [s, None if pages is None else list(pages)]
        assert got == want, (op, iid, ln)


def test_page_manager_demo_sequence():
    """The sequence of the reference's __main__ demo (PageManager.py:164-203)."""
    demo = [t for t in load("page_manager.json") if t["kind"] == "demo"][0]["ops"]
    pm = PageManager(cache_size=32, page_size=4)
    at = 0
    for name, ln in (("A", 5), ("B", 7)):
        r = pm.load_item(name, ln)
        assert [name, ln, [list(r[0]), list(r[1])], pm.get_loaded_lists()] == demo[at]
        at += 1
    pm.access_item("A")
    for name, ln in (("C", 20), ("D", 30)):
        r = _run(pm.load_item, name, ln)
        r = r if isinstance(r, str) else [list(r[0]), list(r[1])]
        assert [name, ln, r, pm.get_loaded_lists()] == demo[at]
        at += 1


def test_fast_order_same_decisions_other_page_numbers():
    """order='fast' evicts the same items and hands out the same NUMBER of pages."""
    rnd = random.Random(3)
    a, b = PageManager(1024, 16), PageManager(1024, 16, order="fast")
    for _ in range(500):
        iid, ln = rnd.randrange(40), rnd.randint(1, 300)
        ra, rb = a.load_item(iid, ln), b.load_item(iid, ln)
        assert len(ra[0]) == len(rb[0]) and ra[1] == rb[1]
        assert len(set(rb[0])) == len(rb[0])
    assert a.get_loaded_lists() == b.get_loaded_lists()
    used = [p for e in b.page_table.values() for p in e["pages"]]
    assert len(used) == len(set(used)) and len(used) + len(b.free_pages) == 64


@pytest.mark.parametrize("case", load("plan_offsets.json"), ids=lambda c: f"p{c['page_size']}n{len(c['id_token_pair'])}")
def test_plan_matches_reference_index_arrays(case, native):
    """src_offsets / dest_offsets as KVCache.shared_data_batch_pages computes them."""
    P = case["page_size"]
    tokens = [p[1] for p in case["id_token_pair"]]
    src, dst = O.reference_offsets(case["cache_pages_list"], tokens, P)
    assert src == case["src_offsets"] and dst == case["dest_offsets"]
    plan = build_plan(case["cache_pages_list"], tokens, P)
    t = plan.table
    assert (t[:, 0] * P).tolist() == case["src_offsets"]
    assert t[:, 3].tolist() == case["dest_offsets"]
    assert plan.n_pages * P == case["total_tokens"]
    assert plan.total_tokens == sum(tokens)
    assert [tuple(r) for r in t.tolist()] == O.plan_records(case["cache_pages_list"], tokens, P)


class _Recorder:
    def __init__(self):
        self.sent = []


@pytest.mark.parametrize("case", load("task_grouping.json"), ids=lambda c: f"n{len(c['tasks'])}")
def test_task_grouping_matches_reference(case):
    """receive_task_info_batch_gprc: same combined tasks (byte-identical
    CombindedTaskInfo messages, same order), same confirmation counts and counters."""
    from bikv_b200.kvcache import KVCache

    kv = KVCache.__new__(KVCache)
    kv.rank, kv.master_port, kv.send_counter, kv.recv_counter = 3, 5000, 0, 0
    kv.workers, kv.stub_factory = {}, None
    sent = []
    kv.send_data_batch = lambda t: sent.append(["RecvKVCacheData", kv._task_info_json_to_pb(t).SerializeToString().hex()])
    kv.receive_data_batch = lambda t: sent.append(["SendKVCacheData", kv._task_info_json_to_pb(t).SerializeToString().hex()])
    tasks = [pb.TaskInfo(**d) for d in case["tasks"]]
    conf = kv.receive_task_info_batch_gprc(tasks)
    assert {str(k): v for k, v in conf.items()} == case["confirmation"]
    assert sent == case["sent"]
    assert (kv.send_counter, kv.recv_counter) == (case["send_counter"], case["recv_counter"])
