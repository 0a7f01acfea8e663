"""The drop-in on the reference's REAL classes (oracle/_ref): `manager.set/apply` -> `pack_model` ->
`generate(past_key_values=PagedQuantCache)` -> `unpack_model` -> `manager.restore()` on
`Qwen2ForCausalLMCompress` / `LlamaForCausalLMCompress` (models/qwen2_c/define_qwen2_c.py:22-27,
models/llama_c/define_llama_c.py:24-30), the decode engine built from a live model, the blocks-path
`convert_for_export` + `LLMWrapper` loop, and config 1 at full size.  The reference runs on the host
cores in the same process and is the oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu

TINY = dict(vocab_size=256, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
            num_key_value_heads=1, max_position_embeddings=128, tie_word_embeddings=False)


def make(T, family, seed, dtype=torch.float32, **over):
    torch.manual_seed(seed)
    kw = {**TINY, **over}
    if family == "qwen2":
        model = T.Qwen2ForCausalLMCompress(T.Qwen2ConfigCompress(**kw))
        mgr = T.Qwen2CompressionSchemesManager(model)
    else:
        model = T.LlamaForCausalLMCompress(T.LlamaConfigCompress(**kw))
        mgr = T.LlamaCompressionSchemesManager(model)
    return model.to(dtype).eval(), mgr


def greedy(model, ids, new, cache=None):
    return model.generate(ids, attention_mask=torch.ones_like(ids), max_new_tokens=new, min_new_tokens=new, do_sample=False,
                          pad_token_id=0, eos_token_id=None, past_key_values=cache)


def linears(T, model):
    from transformersurgeon.blocks import LinearCompressed
    return [(n, m) for n, m in model.named_modules() if type(m) is LinearCompressed]


def rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max()).item()


@pytest.mark.parametrize("family", ["qwen2", "llama"])
def test_apply_pack_generate_unpack_restore(cuda, reference, family):
    """The whole user flow, on the reference's own model class, with nothing of the reference modified."""
    T = reference
    from transformer_surgeon_b200 import surgeon, hf_cache
    model, mgr = make(T, family, 31)
    ids = torch.randint(0, 256, (2, 12), generator=torch.Generator().manual_seed(32))
    with torch.no_grad():
        logits_plain = model(input_ids=ids).logits
    n_lin = len(linears(T, model))
    assert n_lin == 2 * 7 + 1                                         # 7 per block + lm_head
    mgr.set("lrd", "rank", 16, criteria=["mlp"])
    mgr.set("lrd", "rank", 32, criteria=["self_attn.q_proj"])
    mgr.set("quantization", "precision", 8, criteria=["self_attn"])
    mgr.set("quantization", "precision", 4, criteria=["mlp"])
    mgr.set("quantization", "granularity", "per_channel", criteria=["self_attn", "mlp"])
    with surgeon.capture_quantization(model) as cap:                  # keeps the codes the reference drops
        mgr.apply(hard=False)
    assert len(cap.codes) == 2 * (7 + 3 + 1)                          # every factor of every quantized layer
    with torch.no_grad():
        ref_logits = model(input_ids=ids).logits                      # the reference, compressed, on the host
        ref_tokens = greedy(model, ids, 32)
    model.cuda()
    assert surgeon.pack_model(model, cuda) == n_lin
    assert len(linears(T, model)) == n_lin                            # type(m) is LinearCompressed, still
    for path, m in linears(T, model):                                 # the kernels run on the captured codes, bit for bit
        rec = cap.codes.get(path + ".weight")
        if rec is not None:
            assert torch.equal(m._tsb200.u.codes().cpu(), rec[0]) and torch.equal(m._tsb200.u.scales.cpu(), rec[1])
            assert m._tsb200.u.bits == (8 if rec[2] == 8 else 4)
    with torch.no_grad():
        out = model(input_ids=ids.cuda()).logits
    assert rel(out.cpu(), ref_logits) < 1e-4
    model.config._attn_implementation = hf_cache.ATTN_NAME
    cache = hf_cache.PagedQuantCache(model.config, batch=2, max_len=64, kv_format="fp32")
    toks = greedy(model, ids.cuda(), 32, cache)
    assert torch.equal(toks.cpu(), ref_tokens)                        # 32 greedy tokens identical
    surgeon.unpack_model(model)
    assert all("forward" not in m.__dict__ and not hasattr(m, "_tsb200") for _, m in linears(T, model))
    model.config._attn_implementation = "sdpa"
    model.cpu()
    mgr.restore()
    assert len(linears(T, model)) == n_lin
    with torch.no_grad():
        assert torch.allclose(model(input_ids=ids).logits, logits_plain, atol=1e-4)   # test/e2e/test_model_families.py:53-70


@pytest.mark.parametrize("captured", [True, False])
def test_engine_from_live_model_binary_and_4bit(cuda, reference, captured):
    """decoder_from_model on a live Llama compress model: binary MLP factors (sign, mean |w|) + 4-bit attention,
    LRD on the MLP; with the codes captured at apply time, and re-derived from the stored floats (binary: the
    common magnitude of a stored row IS the scale).  Packed factors reconstruct the stored weights exactly;
    logits and 32 greedy tokens equal the reference's."""
    T = reference
    from transformer_surgeon_b200 import surgeon
    model, mgr = make(T, "llama", 33)
    ids = torch.randint(0, 256, (2, 12), generator=torch.Generator().manual_seed(34))
    mgr.set("lrd", "rank", 16, criteria=["mlp"])
    mgr.set("quantization", "precision", 4, criteria=["self_attn"])
    mgr.set("quantization", "precision", "binary", criteria=["mlp"])
    mgr.set("quantization", "granularity", "per_channel", criteria=["self_attn", "mlp"])
    if captured:
        with surgeon.capture_quantization(model):
            mgr.apply(hard=False)
    else:
        mgr.apply(hard=False)
    with torch.no_grad():
        ref_logits = model(input_ids=ids).logits[:, -1]
        ref_tokens = greedy(model, ids, 32)
    dec = surgeon.decoder_from_model(model, batch=2, options={"max_cache_len": 64, "cache_impl": "paged_fp32"})
    assert dec.max_seq_len == 64 and dec.cfg.kv_format == "fp32"
    L0 = dec.layers[0]
    assert L0.gate.u.bits == 1 and L0.gate.v.bits == 1 and L0.o.u.bits == 4 and L0.qkv.u.bits == 4
    sd = model.state_dict()
    assert torch.equal(L0.down.v.reconstruct(torch.float32).cpu(), sd["model.layers.0.mlp.down_proj.linear_V.weight"])
    toks, logits = dec.generate(ids, max_new_tokens=32)
    assert rel(logits.cpu(), ref_logits) < 1e-3
    assert torch.equal(toks.cpu(), ref_tokens)


@pytest.mark.parametrize("impl", ["paged_fp32", "paged_int8", "paged_fp8", "paged_nvfp4"])
def test_blocks_path_llmwrapper_contract(cuda, reference, impl):
    """convert_for_export(options={"cache_impl": paged_*}) + LLMWrapper(input_ids, pos_id, caches) against the
    reference's own converted TransformerDecoder driven the way examples/04_cache_impl_export_interface.py:126-139
    drives it (io_scatter caches, one token per call)."""
    T = reference
    from transformersurgeon.utils.convert import convert_for_export as ref_convert
    from transformer_surgeon_b200 import surgeon, blocks_path
    model, mgr = make(T, "qwen2", 35)
    mgr.set("lrd", "rank", 16, criteria=["mlp"])
    mgr.set("quantization", "precision", 8, criteria=["self_attn", "mlp"])
    mgr.set("quantization", "granularity", "per_channel", criteria=["self_attn", "mlp"])
    mgr.apply(hard=False)
    prompt = torch.randint(0, 256, (9,), generator=torch.Generator().manual_seed(36))
    opts = {"use_sdpa": False, "max_cache_len": 48}
    # ---- the reference's loop (export/common.py:158-176 restated around its own decoder: embedding -> decoder -> final layer)
    rdec = ref_convert(model, options={**opts, "cache_impl": "io_scatter"})["text"].eval()
    kcs = [torch.zeros(b.attn.max_cache_length, b.attn.kv_num_heads, b.attn.head_dim) for b in rdec.blocks]
    vcs = [torch.zeros_like(k) for k in kcs]
    emb, head = model.get_input_embeddings(), model.lm_head
    seq, ref_logits = prompt.clone(), []
    with torch.no_grad():
        for pos in range(9 + 16):
            hidden, kcs, vcs = rdec(emb(seq[pos:pos + 1]), pos_id=torch.tensor([pos]), key_caches=kcs, value_caches=vcs)
            lg = head(hidden[-1, :])
            ref_logits.append(lg)
            if pos >= 8:
                seq = torch.cat([seq, lg.argmax(-1, keepdim=True)])
    # ---- this library, same call shape
    with pytest.raises(ValueError):
        surgeon.convert_for_export(model, options={**opts, "cache_impl": "paged_int3"})      # the reference's validation message
    conv = surgeon.convert_for_export(model, options={**opts, "cache_impl": impl})
    wrapper = blocks_path.LLMWrapper(emb, conv["text"], head)
    assert wrapper.cache_impl == impl and wrapper.decoder.max_cache_len == 48 and wrapper.decoder.depth == 2
    caches = blocks_path.build_paged_caches(wrapper.decoder)
    assert len(caches.key_caches) == 2
    out_seq, logits = prompt.clone(), []
    if impl == "paged_fp8":
        with pytest.raises(ValueError):
            wrapper(prompt[:1], torch.tensor([0]), caches)               # scales unset: refuse rather than saturate
        lg, caches = wrapper.prefill(prompt, caches)                     # one pass over the prompt measures them
        logits += [None] * 8 + [lg.clone()]
        start = 9
        out_seq = torch.cat([out_seq, lg.argmax(-1, keepdim=True).cpu()])
    else:
        start = 0
    for pos in range(start, 9 + 16):
        lg, caches = wrapper(out_seq[pos:pos + 1], torch.tensor([pos]), caches)
        logits.append(lg.clone())
        if pos >= 8:
            out_seq = torch.cat([out_seq, lg.argmax(-1, keepdim=True).cpu()])
    assert int(caches.seq_lens[0]) == 25
    if impl == "paged_fp32":
        assert torch.equal(out_seq, seq)                                  # unquantized pages: same greedy tokens
        for a, b in zip(logits, ref_logits):
            assert rel(a.cpu(), b) < 1e-3
    else:
        tol = {"paged_int8": 3e-2, "paged_fp8": 8e-2, "paged_nvfp4": 2.5e-1}[impl]
        assert rel(logits[8].cpu(), ref_logits[8]) < tol                  # prompt logits (the continuations may part ways)


def test_config1_full_size_32_greedy_tokens(cuda, reference):
    """BASELINE config 1 at full size: Qwen2-0.5B architecture (24 layers, hidden 896, 14/2 heads, d 64, MLP 4864,
    vocab 151936, theta 1e6, tied embeddings), seed 0, fp32, every block linear decomposed by the reference's SVD at
    rank 128, batch 1, 128 uniform-random prompt tokens, 32 greedy tokens, dense fp32 KV.  The reference generates
    on the host; the engine must produce the same 32 tokens."""
    T = reference
    from transformer_surgeon_b200 import surgeon
    torch.manual_seed(0)
    cfg = T.Qwen2ConfigCompress(vocab_size=151936, hidden_size=896, intermediate_size=4864, num_hidden_layers=24,
                                num_attention_heads=14, num_key_value_heads=2, max_position_embeddings=32768,
                                rope_theta=1e6, tie_word_embeddings=True)
    model = T.Qwen2ForCausalLMCompress(cfg).eval()
    mgr = T.Qwen2CompressionSchemesManager(model)
    mgr.set("lrd", "rank", 128, criteria=["self_attn", "mlp"])
    mgr.apply(hard=False)
    ids = torch.randint(0, 151936, (1, 128), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        ref_logits = model(input_ids=ids).logits[:, -1]
        ref_tokens = greedy(model, ids, 32)
    dec = surgeon.decoder_from_model(model, batch=1, max_seq_len=176, kv_format="fp32")
    assert dec.layers[0].gate.rank == 128 and dec.layers[0].qkv is None and dec.layers[0].q.rank == 128
    toks, logits = dec.generate(ids, max_new_tokens=32)
    assert rel(logits.cpu(), ref_logits) < 1e-3
    assert torch.equal(toks.cpu(), ref_tokens)


def test_config5_style_qwen25vl_text_tower_mixed_precision(cuda, reference):
    """BASELINE config 5 in miniature on the reference's own class: the language tower of a
    `Qwen2_5_VLForConditionalGenerationCompress` (models/qwen2_5_vl_c/define_qwen2_5_vl_c.py:44-50) with
    NON-HOMOGENEOUS compression - per-layer weight precision 8 / 2 / 4, per-layer MLP rank 25% / full / 50% - set
    through the reference's manager, text-only token ids (the three mrope position rows coincide, so the rotary
    embedding is the 1-D one).  The engine built from the live model packs each layer at its own precision, gives
    the reference's logits and 32 greedy tokens with unquantized pages, and stays close with NVFP4 pages."""
    T = reference
    from transformer_surgeon_b200 import surgeon
    torch.manual_seed(2)
    text = dict(vocab_size=256, hidden_size=256, intermediate_size=512, num_hidden_layers=3, num_attention_heads=2,
                num_key_value_heads=1, max_position_embeddings=128, tie_word_embeddings=False,
                rope_scaling={"type": "mrope", "mrope_section": [16, 24, 24]})
    vis = dict(depth=1, hidden_size=64, intermediate_size=128, num_heads=2, out_hidden_size=256, fullatt_block_indexes=[0])
    model = T.Qwen2_5_VLForConditionalGenerationCompress(T.Qwen2_5_VLConfigCompress(text_config=text, vision_config=vis, vocab_size=256)).eval()
    mgr = T.Qwen2_5_VLCompressionSchemesManager(model)
    bits, ranks = [8, 2, 4], [128, "full", 256]
    for i in range(3):
        mgr.set("quantization", "precision", bits[i], criteria=[[i, "language_model", "mlp"], [i, "language_model", "self_attn"]])
        mgr.set("quantization", "granularity", "per_channel", criteria=[[i, "language_model"]])
        if ranks[i] != "full":
            mgr.set("lrd", "rank", ranks[i], criteria=[[i, "language_model", "mlp"]])
    with surgeon.capture_quantization(model):
        mgr.apply(hard=False)
    ids = torch.randint(0, 256, (2, 12), generator=torch.Generator().manual_seed(3))
    with torch.no_grad():
        ref_logits = model(input_ids=ids).logits[:, -1]
        ref_tokens = greedy(model, ids, 32)
    dec = surgeon.decoder_from_model(model, batch=2, max_seq_len=64, kv_format="fp32")
    got = [(L.o.u.bits, L.gate.u.bits, L.gate.rank) for L in dec.layers]
    assert got == [(8, 8, 128), (2, 2, 0), (4, 4, 256)], got
    assert dec.layers[0].qkv is not None and dec.layers[0].qkv.bias is not None          # Qwen2 q/k/v carry biases
    toks, logits = dec.generate(ids, max_new_tokens=32)
    assert rel(logits.cpu(), ref_logits) < 1e-3
    assert torch.equal(toks.cpu(), ref_tokens)
    dec4 = surgeon.decoder_from_model(model, batch=2, options={"max_cache_len": 64, "cache_impl": "paged_nvfp4"})
    _, logits4 = dec4.generate(ids, max_new_tokens=1)
    assert rel(logits4.cpu(), ref_logits) < 2.5e-1


def test_gptq_codes_through_capture(cuda, reference):
    """The reference's GPTQ method (compression/quantization_methods/gptq.py:7-104) yields codes and scales in the
    same format as `vanilla`; its calibration runs through the manager's own flow (set_calibration_data -> apply).
    The codes are taken at apply time, packed bit for bit, and logits and 32 greedy tokens equal the reference's."""
    T = reference
    from torch.utils.data import DataLoader
    from transformer_surgeon_b200 import surgeon
    model, mgr = make(T, "llama", 35)
    ids = torch.randint(0, 256, (2, 12), generator=torch.Generator().manual_seed(36))
    mgr.set("lrd", "rank", 16, criteria=["mlp"])
    mgr.set("quantization", "precision", 4, criteria=["self_attn", "mlp"])
    mgr.set("quantization", "method", "gptq", criteria=["self_attn", "mlp"])
    mgr.set("quantization", "granularity", "per_channel", criteria=["self_attn", "mlp"])
    g = torch.Generator().manual_seed(37)
    mgr.set_calibration_data(DataLoader([{"input_ids": torch.randint(0, 256, (4, 24), generator=g)} for _ in range(4)], batch_size=None))
    with surgeon.capture_quantization(model) as cap:
        mgr.apply(hard=False)
    assert len(cap.codes) == 2 * (4 + 3 * 2)
    with torch.no_grad():
        ref_logits = model(input_ids=ids).logits
        ref_tokens = greedy(model, ids, 32)
    model.cuda()
    surgeon.pack_model(model, cuda)
    for path, m in linears(T, model):
        rec = cap.codes.get(path + ".weight")
        if rec is not None:
            assert m._tsb200.u.bits == 4
            assert torch.equal(m._tsb200.u.codes().cpu(), rec[0]) and torch.equal(m._tsb200.u.scales.cpu(), rec[1])
    with torch.no_grad():
        out = model(input_ids=ids.cuda()).logits
    assert rel(out.cpu(), ref_logits) < 1e-4
    surgeon.unpack_model(model)
    dec = surgeon.decoder_from_model(model.cpu(), batch=2, options={"max_cache_len": 64, "cache_impl": "paged_fp32"})
    assert dec.layers[0].o.u.bits == 4 and dec.layers[0].down.v.bits == 4
    toks, _ = dec.generate(ids, max_new_tokens=32)
    assert torch.equal(toks.cpu(), ref_tokens)


def test_packed_codes_in_the_checkpoint(cuda, reference, tmp_path):
    """Packed codes as state_dict buffers: they survive manager.prepare_for_save() and save_pretrained, a model
    built by from_pretrained ignores them, and load_packed_checkpoint attaches the kernels from the file alone -
    the same containers bit for bit, the same logits bit for bit as the model that was saved."""
    T = reference
    from safetensors.torch import load_file
    from transformer_surgeon_b200 import surgeon
    model, mgr = make(T, "llama", 38)
    ids = torch.randint(0, 256, (2, 12), generator=torch.Generator().manual_seed(39))
    mgr.set("lrd", "rank", 16, criteria=["mlp"])
    mgr.set("quantization", "precision", 4, criteria=["self_attn"])
    mgr.set("quantization", "precision", 2, criteria=["mlp"])
    mgr.set("quantization", "granularity", "per_channel", criteria=["self_attn", "mlp"])
    with surgeon.capture_quantization(model):
        mgr.apply(hard=False)
    model.cuda()
    n = surgeon.pack_model(model, cuda)
    with torch.no_grad():
        out = model(input_ids=ids.cuda()).logits
    assert surgeon.register_packed_buffers(model) == n
    mgr.prepare_for_save()                                            # utils/manager.py:843-894
    keys = [k for k in model.state_dict() if "._tsb200_" in k]
    assert len(keys) >= 4 * n
    model.save_pretrained(tmp_path)
    stored = load_file(str(tmp_path / "model.safetensors"))
    assert all(k in stored for k in keys)
    fresh = T.LlamaForCausalLMCompress.from_pretrained(tmp_path).eval().cuda()   # rebuilt from config.compression_config
    assert not any("._tsb200_" in k for k in fresh.state_dict())
    assert surgeon.load_packed_checkpoint(fresh, tmp_path, cuda) == n
    for (pa, a), (pb, b) in zip(linears(T, model), linears(T, fresh)):
        assert pa == pb and a._tsb200.u.bits == b._tsb200.u.bits
        assert torch.equal(a._tsb200.u.data, b._tsb200.u.data)
        assert (a._tsb200.u.scales is None and b._tsb200.u.scales is None) or torch.equal(a._tsb200.u.scales, b._tsb200.u.scales)
        assert (a._tsb200.v is None) == (b._tsb200.v is None)
    with torch.no_grad():
        out2 = fresh(input_ids=ids.cuda()).logits
    assert torch.equal(out2, out)
    surgeon.unpack_model(model)
    assert not any("._tsb200_" in k for k in model.state_dict())
