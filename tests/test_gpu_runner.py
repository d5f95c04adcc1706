"""The native runner q35run (C++ against the C ABI) on case directories: results bit-identical to the Python host's."""
import os
import subprocess

import pytest
import torch

from _cases import gdn_step_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def runner():
    from ax_dsl_kernels_b200 import build
    build.build()
    return build.RUNNER


def test_route_from_files(runner, golden, tmp_path):
    import ax_dsl_kernels_b200 as q35
    from ax_dsl_kernels_b200 import casefile
    f = golden("route")
    ids, rw = q35.route(f["logits"].cuda(), 8)
    casefile.dump_case(tmp_path, dict(logits=f["logits"]), dict(ids=ids, rw=rw))
    r = subprocess.run([runner, "moe.route", str(tmp_path), "5", "--check", "2"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "check: 2 runs, 0 differing outputs" in r.stdout and "device status 0" in r.stdout
    assert torch.equal(casefile.read_output(tmp_path, "ids", ids), ids.cpu())
    assert torch.equal(casefile.read_output(tmp_path, "rw", rw), rw.cpu())


def test_gdn_step_in_place_state_from_files(runner, tmp_path):
    """state_out aliased onto state_in (Q35RUN_ALIAS), as the reference's runner aliases recurrent state"""
    import ax_dsl_kernels_b200 as q35
    from ax_dsl_kernels_b200 import casefile
    q, k, v, g, beta, state = gdn_step_case(B=4, NK=2, NV=4, seed=12)
    ins = dict(q=q[:, 0], k=k[:, 0], v=v[:, 0], g=g[:, 0], beta=beta[:, 0], state_in=state)
    o, s1 = q35.gdn_recurrent_step(*(t.contiguous().cuda() for t in ins.values()))
    casefile.dump_case(tmp_path, {n: t.contiguous() for n, t in ins.items()}, dict(o=o, state_out=s1))
    env = dict(os.environ, Q35RUN_ALIAS="state_out:state_in")
    r = subprocess.run([runner, "gdn.step", str(tmp_path), "0", "--check", "3"], capture_output=True, text=True, env=env)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "in place of input state_in" in r.stdout and "check: 3 runs, 0 differing outputs" in r.stdout
    assert torch.equal(casefile.read_output(tmp_path, "o", o), o.cpu())
    assert torch.equal(casefile.read_output(tmp_path, "state_out", s1), s1.cpu())


def test_workspace_role_and_contract_error(runner, golden, tmp_path):
    import ax_dsl_kernels_b200 as q35
    from ax_dsl_kernels_b200 import casefile
    from ax_dsl_kernels_b200.moe import lm_head
    f = golden("lm_head")
    logits, token = lm_head(f["x"].cuda(), f["packed"].cuda(), f["scale"].cuda())
    casefile.dump_case(tmp_path, dict(x=f["x"], w=f["packed"], s=f["scale"]), dict(logits=logits, token=token))
    r = subprocess.run([runner, "lm_head", str(tmp_path), "3"], capture_output=True, text=True)
    assert r.returncode == 0 and "(scratch)" in r.stdout, r.stdout + r.stderr
    assert torch.equal(casefile.read_output(tmp_path, "logits", logits), logits.cpu())
    assert torch.equal(casefile.read_output(tmp_path, "token", token), f["token"])
    # a wrong shape is a status with a message, not a crash
    bad = tmp_path / "bad"
    casefile.dump_case(bad, dict(x=f["x"], w=f["packed"][:, :100], s=f["scale"]), dict(logits=logits))
    r = subprocess.run([runner, "lm_head", str(bad), "0"], capture_output=True, text=True)
    assert r.returncode == 1 and "lm_head" in r.stderr
    assert q35.device_status() == 0


def test_manifest_roles_run_with_the_reference_shapes(tmp_path):
    """moe.combine_t512 and lm_head exactly as the reference's 35B manifest declares them (tensor names, dtype codes,
    byte counts; lm_head's output under the manifest's name `out`), against the oracle"""
    import ax_dsl_kernels_b200 as q35
    from ax_dsl_kernels_b200 import manifest
    from conftest import assert_parity, rel_rms_err
    from oracle import codecs, moe as omoe
    m = manifest.load(os.path.join(os.path.dirname(__file__), "golden", "manifest_35b_roles.json"))
    g = torch.Generator().manual_seed(6)
    T, K, R, H = 512, 8, 32768, 2048
    base = torch.randn((T, H), generator=g).to(torch.bfloat16)
    sout = torch.randn((R, H), generator=g).to(torch.bfloat16)
    loc = torch.randperm(R, generator=g)[:K * T].reshape(K, T).to(torch.int32)
    out = torch.empty((T, H), dtype=torch.bfloat16).cuda()
    manifest.run_role(m, "moe.combine_t512", dict(base=base.cuda(), loc=loc.cuda(), sout=sout.cuda(), out=out))
    assert_parity(out.cpu(), omoe.combine(base, loc, sout), tol=1e-3, bf16_step=True)
    with pytest.raises(ValueError):
        manifest.run_role(m, "moe.combine_t512", dict(base=base[:8].cuda(), loc=loc.cuda(), sout=sout.cuda(), out=out))

    N = 248320
    pk, sc = codecs.random_mxfp4((N, H), g, -8, 0)
    x = torch.randn((1, H), generator=g).to(torch.bfloat16)
    logits = torch.empty((1, N), dtype=torch.float32).cuda()
    # the manifest declares w as logical FP4 [N, K] (code 15); the bytes are the packed pairs
    manifest.run_role(m, "lm_head", dict(x=x.cuda(), w=pk.cuda(), s=sc.cuda(), out=logits))
    assert rel_rms_err(logits.cpu(), codecs.lm_head_logits(x, pk, sc)[0]) <= 2e-2
    assert q35.device_status() == 0


def test_four_host_threads_run_replicas_bitwise_equal(runner, tmp_path):
    """q35run --par: four host threads, a stream and a buffer set each, barrier per round; every replica's outputs
    equal replica 0's (what the reference's par_test.cc checks across its four cores)"""
    import ax_dsl_kernels_b200 as q35
    from ax_dsl_kernels_b200 import casefile
    from _cases import paged_case
    q, cache, indptr, indices, last, _ = paged_case([300, 17, 1500, 64])
    out = q35.paged_attention_decode(q.cuda(), cache.cuda(), indptr.cuda(), indices.cuda(), last.cuda())
    casefile.dump_case(tmp_path, dict(q=q, paged_kv_cache=cache, indptr=indptr, indices=indices, last_page_len=last),
                       dict(out=out))
    r = subprocess.run([runner, "--par", "4", "attn.paged_decode", str(tmp_path), "--rounds", "8"], capture_output=True,
                       text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "RESULT par=4 rounds=8" in r.stdout and "differing=0 run_failures=0 device_status=0" in r.stdout


def test_roles_alternated_with_poisoned_outputs(runner, golden, tmp_path):
    """q35run --alt: three roles called in turn for several rounds, outputs filled with 0xFF before every call from
    round 1 on and compared with round 0 (mc_alt.cc with SENTINEL=1): no role leaves output bytes unwritten"""
    import ax_dsl_kernels_b200 as q35
    from ax_dsl_kernels_b200 import casefile
    from _cases import paged_case
    f = golden("route")
    ids, rw = q35.route(f["logits"].cuda(), 8)
    d1, d2, d3 = tmp_path / "route", tmp_path / "attn", tmp_path / "gdn"
    casefile.dump_case(d1, dict(logits=f["logits"]), dict(ids=ids, rw=rw))
    q, cache, indptr, indices, last, _ = paged_case([70, 1, 200])
    out = q35.paged_attention_decode(q.cuda(), cache.cuda(), indptr.cuda(), indices.cuda(), last.cuda())
    casefile.dump_case(d2, dict(q=q, paged_kv_cache=cache, indptr=indptr, indices=indices, last_page_len=last),
                       dict(out=out))
    gq, gk, gv, gg, gb, st = gdn_step_case(B=2, NK=2, NV=4, seed=3)
    ins = dict(q=gq[:, 0], k=gk[:, 0], v=gv[:, 0], g=gg[:, 0], beta=gb[:, 0], state_in=st)
    o, s1 = q35.gdn_recurrent_step(*(t.contiguous().cuda() for t in ins.values()), state_out=torch.empty_like(st).cuda())
    casefile.dump_case(d3, {n: t.contiguous() for n, t in ins.items()}, dict(o=o, state_out=s1))
    r = subprocess.run([runner, "--alt", "moe.route", str(d1), "attn.paged_decode", str(d2), "gdn.step", str(d3),
                        "--rounds", "4"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.count("fails=0 mismatches=0") == 3 and "device_status=0" in r.stdout
