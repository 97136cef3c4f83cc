"""The reference's own caller on this library: `pie_worker.model.llama3.ForwardPass` (unmodified, imported from
a checkout named by the environment) with `pie_b200.ops` standing where it imports `flashinfer`
(pie/src/pie_worker/model/llama3.py:18-21).

Set PIE_REFERENCE_SRC to `<reference checkout>/pie/src` (the folder that holds `pie_worker/`); without it the
test skips.  Nothing else in the suite reads the reference tree.

What runs is the reference's code path end to end: `Batch` turns wire bytes into tensors
(pie/src/pie_worker/batching.py:28-239), `ForwardPass.transform` derives metadata, plans the prefill wrapper
with the `custom_mask` `Batch` produced or the decode wrapper, and runs two layers — RoPE on strided views of
the fused QKV projection, append, attention — eagerly and through its CUDA-graph bins
(llama3.py:229-313,588-823,866-956).  Every operator call it makes is recorded by a thin layer around the
shim and checked against the CPU oracle on the very tensors it was given; the graph path must then leave the
same pools as the eager path, bit for bit.
"""
import os
import sys
import types

import numpy as np
import pytest
import torch

from oracle import paged_kv_ref as R
from util import ulp_diff_bf16

REF = os.environ.get("PIE_REFERENCE_SRC", "")
HAVE_REF = os.path.isdir(os.path.join(REF, "pie_worker"))

pytestmark = [
    pytest.mark.gpu,
    pytest.mark.skipif(not HAVE_REF, reason="PIE_REFERENCE_SRC does not name <reference checkout>/pie/src"),
]

LAYERS, HQ, HKV, D, HIDDEN, MLP, VOCAB, PAGE = 2, 32, 8, 128, 512, 1024, 64, 16
MAX_PAGES = 96


class Log:
    """What the reference's caller asked of the operator module, in call order."""

    def __init__(self):
        self.on = True
        self.calls = []
        self.plan = None

    def recording(self):
        return self.on and not torch.cuda.is_current_stream_capturing()


def host(x):
    return x.detach().cpu().numpy() if isinstance(x, torch.Tensor) else np.asarray(x)


def make_shim(log):
    """A module object that is `pie_b200.ops` plus recording, installed under the name the reference imports."""
    import pie_b200.ops as ops

    mod = types.ModuleType("flashinfer")
    mod.__path__ = []  # a package, so that `flashinfer.sampling` resolves
    for name in dir(ops):
        if not name.startswith("_"):
            setattr(mod, name, getattr(ops, name))

    def rope(**kw):
        if not log.recording():
            return ops.apply_llama31_rope_pos_ids_inplace(**kw)
        before = (kw["q"].detach().cpu().clone(), kw["k"].detach().cpu().clone())
        assert not kw["q"].is_contiguous(), "the reference hands over views of the fused projection"
        ops.apply_llama31_rope_pos_ids_inplace(**kw)
        log.calls.append(("rope", before, (kw["q"].detach().cpu().clone(), kw["k"].detach().cpu().clone()),
                          host(kw["pos_ids"]), {k: v for k, v in kw.items() if k not in ("q", "k", "pos_ids")}))

    def append(**kw):
        if not log.recording():
            return ops.append_paged_kv_cache(**kw)
        pool_before = kw["paged_kv_cache"].detach().cpu().clone()
        ops.append_paged_kv_cache(**kw)
        log.calls.append(("append", pool_before, kw["paged_kv_cache"].detach().cpu().clone(),
                          kw["append_key"].detach().cpu().clone(), kw["append_value"].detach().cpu().clone(),
                          host(kw["batch_indices"]), host(kw["positions"]), host(kw["kv_indices"]),
                          host(kw["kv_indptr"]), host(kw["kv_last_page_len"])))

    def seq_lens(*a, **kw):
        out = ops.get_seq_lens(*a, **kw)
        if log.recording():
            log.calls.append(("seq_lens", host(a[0]), host(a[1]), a[2], host(out)))
        return out

    def batch_pos(**kw):
        out = ops.get_batch_indices_positions(**kw)
        if log.recording():
            log.calls.append(("batch_pos", host(kw["append_indptr"]), host(kw["seq_lens"]), kw["nnz"],
                              host(out[0]), host(out[1])))
        return out

    class Decode(ops.BatchDecodeWithPagedKVCacheWrapper):
        def plan(self, **kw):
            if log.recording():
                self._seen = dict(indptr=host(kw["indptr"]), indices=host(kw["indices"]),
                                  last=host(kw["last_page_len"]))
            return super().plan(**kw)

        def run(self, q, kv):
            out = super().run(q, kv)
            if log.recording():
                log.calls.append(("decode", q.detach().cpu().clone(), kv.detach().cpu().clone(), dict(self._seen),
                                  out.detach().cpu().clone()))
            return out

    class Prefill(ops.BatchPrefillWithPagedKVCacheWrapper):
        def plan(self, **kw):
            if log.recording():
                self._seen = dict(qo=host(kw["qo_indptr"]), indptr=host(kw["paged_kv_indptr"]),
                                  indices=host(kw["paged_kv_indices"]), last=host(kw["paged_kv_last_page_len"]),
                                  mask=None if kw.get("custom_mask") is None else host(kw["custom_mask"]))
            return super().plan(**kw)

        def run(self, q, kv):
            out = super().run(q, kv)
            if log.recording():
                log.calls.append(("prefill", q.detach().cpu().clone(), kv.detach().cpu().clone(), dict(self._seen),
                                  out.detach().cpu().clone()))
            return out

    mod.apply_llama31_rope_pos_ids_inplace = rope
    mod.append_paged_kv_cache = append
    mod.get_seq_lens = seq_lens
    mod.get_batch_indices_positions = batch_pos
    mod.BatchDecodeWithPagedKVCacheWrapper = Decode
    mod.BatchPrefillWithPagedKVCacheWrapper = Prefill

    sampling = types.ModuleType("flashinfer.sampling")  # imported by the reference's model code, not on this path

    def not_on_this_path(*a, **k):
        raise AssertionError("sampling is outside the paged-KV path")

    for name in ("sampling_from_probs", "top_p_sampling_from_probs", "top_k_sampling_from_probs",
                 "min_p_sampling_from_probs", "top_k_top_p_sampling_from_probs"):
        setattr(sampling, name, not_on_this_path)
    mod.sampling = sampling
    return mod, sampling


@pytest.fixture
def reference(monkeypatch):
    """The reference's modules imported fresh over the shim; everything is put back afterwards."""
    log = Log()
    mod, sampling = make_shim(log)
    for name in [m for m in sys.modules if m == "pie_worker" or m.startswith("pie_worker.")]:
        monkeypatch.delitem(sys.modules, name)
    monkeypatch.setitem(sys.modules, "flashinfer", mod)
    monkeypatch.setitem(sys.modules, "flashinfer.sampling", sampling)
    monkeypatch.syspath_prepend(REF)
    import pie_worker.model.llama3 as llama3
    from pie_worker.batching import Batch
    from pie_worker.config import RuntimeConfig
    from pie_worker.loader import WeightStore
    assert llama3.ops is mod
    yield types.SimpleNamespace(llama3=llama3, Batch=Batch, RuntimeConfig=RuntimeConfig, WeightStore=WeightStore,
                                log=log)
    for name in [m for m in sys.modules if m == "pie_worker" or m.startswith("pie_worker.")]:
        monkeypatch.delitem(sys.modules, name, raising=False)


def build_engine(ref, use_graphs):
    dev = torch.device("cuda", 0)
    mc = ref.llama3.ModelConfig(
        num_vocabs=VOCAB, num_layers=LAYERS, num_q_heads=HQ, num_kv_heads=HKV, dim_head=D, dim_hidden=HIDDEN,
        dim_mlp=MLP, rms_norm_eps=1e-5, rope_factor=8.0, rope_high_frequency_factor=4.0,
        rope_low_frequency_factor=1.0, rope_original_max_position_embeddings=8192, rope_theta=500000.0,
        tie_word_embeddings=True)
    rc = ref.RuntimeConfig(
        hf_repo="none", cache_dir="", kv_page_size=PAGE, max_dist_size=32, max_num_embeds=8, max_batch_tokens=4096,
        max_batch_size=16, max_num_adapters=1, max_adapter_rank=1, gpu_mem_utilization=0.5, random_seed=0,
        use_cuda_graphs=use_graphs, tensor_parallel_size=1, telemetry_enabled=False, telemetry_endpoint="",
        telemetry_service_name="", adapter_path="", max_num_kv_pages=MAX_PAGES, devices=[dev], rank=0,
        activation_dtype=torch.bfloat16, weight_dtype="auto")
    g = torch.Generator().manual_seed(5)

    def w(*shape, scale):
        return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).to(dev)

    ws = ref.WeightStore()
    ws.put("embed_token", w(VOCAB, HIDDEN, scale=1.0))
    ws.put("norm_last", torch.ones(HIDDEN, dtype=torch.bfloat16, device=dev))
    for i in range(LAYERS):
        ws.put(f"layers.{i}.norm_attn", torch.ones(HIDDEN, dtype=torch.bfloat16, device=dev))
        ws.put(f"layers.{i}.norm_mlp", torch.ones(HIDDEN, dtype=torch.bfloat16, device=dev))
        ws.put(f"layers.{i}.proj_qkv", w((HQ + 2 * HKV) * D, HIDDEN, scale=HIDDEN ** -0.5))
        ws.put(f"layers.{i}.proj_o", w(HIDDEN, HQ * D, scale=(HQ * D) ** -0.5))
        ws.put(f"layers.{i}.proj_gate_up", w(2 * MLP, HIDDEN, scale=HIDDEN ** -0.5))
        ws.put(f"layers.{i}.proj_down", w(HIDDEN, MLP, scale=MLP ** -0.5))
    engine = ref.llama3.ForwardPass(mc, rc, ws)
    pools = ref.llama3.create_kv_cache(mc, rc)
    return engine, pools, dev


def u32(x):
    return np.asarray(x, dtype=np.uint32).tobytes()


def f32(x):
    return np.asarray(x, dtype=np.float32).tobytes()


class Requests:
    """Page lists of the test's requests, dealt from a seeded permutation of the pool's page ids."""

    def __init__(self, prompt_lens, seed=3):
        self.free = list(np.random.default_rng(seed).permutation(MAX_PAGES))
        self.tokens = [0] * len(prompt_lens)
        self.pages = [[] for _ in prompt_lens]

    def wire(self, new_tokens, single_token_mode):
        """Grow every request by `new_tokens[r]` and return the wire form of the step
        (runtime/src/model/request.rs:250-298; causal run lengths, one run per query token)."""
        qo, ptr, idx, last, runs, rptr, pos = [0], [0], [], [], [], [0], []
        for r, m in enumerate(new_tokens):
            ctx = self.tokens[r]
            self.tokens[r] = ctx + m
            while len(self.pages[r]) * PAGE < self.tokens[r]:
                self.pages[r].append(int(self.free.pop(0)))
            idx += self.pages[r]
            ptr.append(ptr[-1] + len(self.pages[r]))
            last.append((self.tokens[r] - 1) % PAGE + 1)
            qo.append(qo[-1] + m)
            for j in range(m):
                pos.append(ctx + j)
                runs.append(ctx + j + 1)
                rptr.append(rptr[-1] + 1)
        nreq, ntok = len(new_tokens), qo[-1]
        return {
            "token_ids": u32(np.arange(ntok) % VOCAB), "position_ids": u32(pos), "kv_page_indices": u32(idx),
            "kv_page_indptr": u32(ptr), "kv_last_page_lens": u32(last), "qo_indptr": u32(qo),
            "flattened_masks": u32(runs), "mask_indptr": u32(rptr), "single_token_mode": single_token_mode,
            "adapter_indices": [None] * nreq, "adapter_seeds": [None] * nreq,
            "sampler_temperatures": f32([]), "sampler_top_k": u32([]), "sampler_top_p": f32([]),
            "sampler_min_p": f32([]), "sampler_types": u32([]), "request_num_samplers": u32([0] * nreq),
            "flat_output_token_indices": u32([]), "output_token_indptr": u32([0] * (nreq + 1)),
        }


def run_steps(ref, use_graphs, prompt_lens, decode_steps):
    """Prefill + decode steps through the reference's `Batch` and `ForwardPass.transform`."""
    engine, pools, dev = build_engine(ref, use_graphs)
    if use_graphs:
        ref.log.on = False  # the warm-up runs every bin on dummy tables; nothing to compare there
        engine.warmup_cuda_graphs(pools)
        ref.log.on = True
    reqs = Requests(prompt_lens)
    g = torch.Generator().manual_seed(17)
    outs = []
    for step in range(1 + decode_steps):
        decode = step > 0
        args = reqs.wire([1] * len(prompt_lens) if decode else prompt_lens, decode)
        batch = ref.Batch(args, kv_page_size=PAGE, max_dist_size=32, adapters={})
        inputs = batch.get_model_inputs(dev)
        n = int(inputs["qo_indptr"][-1])
        embeds = torch.randn(n, HIDDEN, generator=g).to(torch.bfloat16).to(dev)
        hidden = engine.transform(
            input_embeds=embeds, position_ids=inputs["position_ids"], qo_indptr=inputs["qo_indptr"],
            kv_cache_at_layer=pools, kv_page_indices=inputs["kv_page_indices"],
            kv_page_indptr=inputs["kv_page_indptr"], kv_last_page_lens=inputs["kv_last_page_lens"],
            custom_mask=inputs["custom_mask"], single_token_inference_mode=inputs["single_token_inference_mode"],
            adapter_subpass=None, total_pages_cpu=inputs.get("total_pages_cpu", 0))
        torch.cuda.synchronize()
        outs.append(hidden.detach().cpu().clone())
    return outs, [p.detach().cpu().clone() for p in pools]


def check_calls(calls):
    """Every recorded operator call against the CPU oracle on the tensors the caller passed."""
    seen = {}
    for c in calls:
        kind = c[0]
        seen[kind] = seen.get(kind, 0) + 1
        if kind == "seq_lens":
            _, ptr, last, page, out = c
            assert np.array_equal(out, R.get_seq_lens(ptr, last, page))
        elif kind == "batch_pos":
            _, qo, sl, nnz, bi, pos = c
            want_bi, want_pos = R.get_batch_indices_positions(qo, sl, nnz)
            assert np.array_equal(bi, want_bi) and np.array_equal(pos, want_pos)
        elif kind == "rope":
            _, (q0, k0), (q1, k1), pos, kw = c
            inv = R.rope_inv_freq(D, kw["rope_theta"], "llama31", kw["rope_scale"], kw["low_freq_factor"],
                                  kw["high_freq_factor"], kw["old_context_len"])
            cs, sn = R.rope_cos_sin(pos, inv)
            assert ulp_diff_bf16(q1, R.apply_rope(q0, cs, sn)) <= 1
            assert ulp_diff_bf16(k1, R.apply_rope(k0, cs, sn)) <= 1
        elif kind == "append":
            _, before, after, k, v, bi, pos, idx, ptr, last = c
            R.append_paged_kv_cache(k, v, bi, pos, before, idx, ptr, last)
            assert torch.equal(before.view(torch.int16), after.view(torch.int16))
        elif kind == "decode":
            _, q, pool, t, out = c
            want = R.decode_attention(q, pool, t["indptr"], t["indices"], t["last"])
            assert (out.float() - want.float()).abs().max().item() <= 2e-2
        elif kind == "prefill":
            _, q, pool, t, out = c
            assert t["mask"] is not None, "the reference plans its prefill wrapper with the mask Batch derived"
            want = R.prefill_attention(q, pool, t["qo"], t["indptr"], t["indices"], t["last"], custom_mask=t["mask"])
            assert (out.float() - want.float()).abs().max().item() <= 2e-2
    return seen


def test_reference_forward_pass_runs_on_this_library_eagerly_and_through_its_graph_bins(reference):
    prompts = [37, 16, 5, 70]  # four requests: one of the reference's graph bins, so no padding rows
    steps = 3
    eager_out, eager_pools = run_steps(reference, False, prompts, steps)
    seen = check_calls(reference.log.calls)
    assert seen["prefill"] == LAYERS and seen["decode"] == LAYERS * steps
    assert seen["rope"] == seen["append"] == LAYERS * (1 + steps)
    assert seen["seq_lens"] == seen["batch_pos"] == 1 + steps
    assert all(torch.isfinite(o.float()).all() for o in eager_out)

    reference.log.calls.clear()
    graph_out, graph_pools = run_steps(reference, True, prompts, steps)
    check_calls(reference.log.calls)  # the prefill step and the metadata calls still run eagerly
    # The prefill step runs eagerly in both engines.  For the decode steps the reference's captured graph leaves
    # its result in a tensor of the graph's own memory pool, and `_run_layers_graphed` hands back the static
    # INPUT rows (llama3.py:396-411,956), so its hidden states say nothing about the operators.  The pools
    # do: the second layer's new K / V rows are computed, inside the graph, from the first layer's attention
    # output over the page tables of that step.
    assert torch.equal(eager_out[0].view(torch.int16), graph_out[0].view(torch.int16))
    for a, b in zip(eager_pools, graph_pools):
        # the scratch page (the last one) is where the warm-up wrote its dummy rows
        assert torch.equal(a[:MAX_PAGES].view(torch.int16), b[:MAX_PAGES].view(torch.int16))
    assert not torch.equal(eager_pools[1][:MAX_PAGES], torch.zeros_like(eager_pools[1][:MAX_PAGES]))
