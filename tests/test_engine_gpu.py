"""The engine against the plain implementation, in float32 and in bfloat16, under every schedule:
each request alone and whole; its last 32 tokens one by one; batches of unequal lengths whose shorter
requests end earlier, batch after batch so that slots and pages are used again; long decoding; the
first tokens of a sequence; greedy generation through the entry point; sampling."""

from __future__ import annotations

import numpy as np
import pytest
import torch

import tiny
from closeness import check
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

# float32, decided before the first run: the engine and the plain code differ by summation order only (the largest
# difference a B200 showed over all tests of this file: 1.2e-6 on logits up to 1.4).
# bfloat16: weights are compared rounded alike, activations and cache entries are rounded in the engine only. The
# bound was set at about twice the largest difference the tiny configurations showed on a B200 (0.0106 on logits up
# to 2.1; the odd head sizes added later reach 0.0132 on logits up to 2.4; tests/closeness.py prints what a run saw),
# as an absolute bound with no relative part: a key rounded twice or a gain applied in bfloat16 lies outside it.
TOL = {"fp32": dict(rtol=1e-4, atol=2e-5), "bf16": dict(rtol=0.0, atol=1.7e-2)}


def load(folder, dtype, max_tokens=4096, **kw):
    import sleuth_b200 as sb
    cfg = plain.read_model(folder)[0]
    return sb.load(folder, dtype=dtype, max_seq_len=cfg["max_position_embeddings"], max_tokens=max_tokens, **kw)


def oracle(folder, dtype):
    cfg, w = plain.read_model(folder)
    cache = {}

    def f(ids):
        key = tuple(ids)
        if key not in cache:
            cache[key] = plain.logits(cfg, w, list(ids), round_weights_to_bf16=(dtype == "bf16"))
        return cache[key]
    return f


def requests_for(name, lengths, seed=0):
    rng = np.random.default_rng(seed + tiny.SEEDS[name])
    return [rng.integers(0, tiny.CONFIGS[name]["vocab_size"], size=n).tolist() for n in lengths]


LENGTHS = {"A": [5, 11, 17, 70], "B": [1, 7, 23, 40, 130], "C": [3, 64, 65, 150, 33], "D": [40, 1, 200, 129],
           "E": [10, 140, 300, 129], "F": [10, 140, 300, 129, 65], "G": [33, 1, 200, 700]}


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F", "G"])
def test_each_request_alone_and_whole(name, dtype, model_folders):
    eng, ref = load(model_folders[name], dtype), oracle(model_folders[name], dtype)
    for ids in requests_for(name, LENGTHS[name]):
        (slot,) = eng.open(1)
        got = eng.step([(slot, ids, tuple(range(len(ids))))]).cpu()
        eng.close([slot])
        check(got, ref(ids), TOL[dtype], "engine " + dtype)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F", "G"])
def test_last_32_tokens_one_by_one(name, dtype, model_folders):
    eng, ref = load(model_folders[name], dtype), oracle(model_folders[name], dtype)
    for ids in requests_for(name, [n for n in LENGTHS[name] if n > 32] + [33]):
        cut = len(ids) - 32
        (slot,) = eng.open(1)
        rows = [eng.step([(slot, ids[:cut], (cut - 1,))]).cpu()]
        for t in ids[cut:]:
            rows.append(eng.step([(slot, [t], (0,))]).cpu().clone())
        eng.close([slot])
        check(torch.cat(rows), ref(ids)[cut - 1:], TOL[dtype], "engine " + dtype)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F", "G"])
def test_unequal_batches_one_after_another_reuse_slots(name, dtype, model_folders):
    """Three batches through a cache with room for one batch only. Within a batch the requests have unequal
    prompts and unequal numbers of decoded tokens, so the shorter ones end earlier; the next batch gets
    the same slots and pages, still full of the previous batch's keys."""
    max_tokens = 64 * 8
    eng, ref = load(model_folders[name], dtype, max_tokens=max_tokens), oracle(model_folders[name], dtype)
    ctx = tiny.CONFIGS[name]["max_position_embeddings"]
    plans = [[(100, 20), (60, 3), (5, 27)], [(1, 12), (64, 1), (63, 2), (30, 30)], [(90, 9), (2, 40)]]
    used_slots = []
    for b, plan in enumerate(plans):
        plan = [(p, d) for p, d in plan if p + d <= ctx]
        reqs = requests_for(name, [p + d for p, d in plan], seed=b)
        slots = eng.open(len(reqs))
        used_slots.append(set(slots))
        got = {i: [] for i in range(len(reqs))}
        out = eng.step([(s, ids[:p], (p - 1,)) for s, ids, (p, d) in zip(slots, reqs, plan)]).cpu()
        for i in range(len(reqs)):
            got[i].append(out[i])
        live = list(range(len(reqs)))
        k = 0
        while live:
            live = [i for i in live if k < plan[i][1]]
            if not live:
                break
            out = eng.step([(slots[i], [reqs[i][plan[i][0] + k]], (0,)) for i in live]).cpu()
            for j, i in enumerate(live):
                got[i].append(out[j].clone())
            done = [i for i in live if k + 1 >= plan[i][1]]
            eng.close([slots[i] for i in done])                       # a shorter request ends earlier
            live = [i for i in live if i not in done]
            k += 1
        for i, ids in enumerate(reqs):
            p = plan[i][0]
            check(torch.stack(got[i]), ref(ids)[p - 1:], TOL[dtype], "engine " + dtype)
    assert used_slots[1] & used_slots[0] and used_slots[2] & used_slots[0]
    assert eng.cache.book.pages_in_use() == [0] * eng.cache.n_groups and eng.cache.book.free_slots == eng.cache.max_slots


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_long_decoding(dtype, model_folders):
    """600 tokens decoded one by one after a short prompt: positions cross nine pages, the decode step runs
    as a captured graph from its second occurrence on, and the window layers of C drop pages on the way."""
    for name, total in (("D", 640), ("C", 330), ("F", 400), ("G", 640)):
        eng, ref = load(model_folders[name], dtype, max_tokens=1024), oracle(model_folders[name], dtype)
        (ids,) = requests_for(name, [total], seed=5)
        (slot,) = eng.open(1)
        eng.step([(slot, ids[:7], ())])
        look_at = {7, 8, 63, 64, 65, 127, 128, 200, 319, 320, total - 1}
        for t in range(7, total):
            out = eng.step([(slot, [ids[t]], (0,))])
            if t in look_at:
                check(out.cpu()[0], ref(ids)[t], TOL[dtype], "engine " + dtype)
        if name in ("C", "F"):
            win = [g for g in eng.cache.book.groups if g.window][0]
            assert (win.table[slot] >= 0).sum() <= (2 if name == "C" else 3)     # 40 (70) keys never need more pages
        eng.close([slot])


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "F", "G"])
def test_first_tokens(name, dtype, model_folders):
    eng, ref = load(model_folders[name], dtype), oracle(model_folders[name], dtype)
    (ids,) = requests_for(name, [4], seed=9)
    (slot,) = eng.open(1)
    rows = [eng.step([(slot, [t], (0,))]).cpu().clone() for t in ids]       # position 0 on: no prompt step at all
    eng.close([slot])
    check(torch.cat(rows), ref(ids), TOL[dtype], "engine " + dtype)


def _odd(hidden, inter, layers, heads, kv_heads, head_dim, vocab, bias, tied, window=None):
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=vocab, hidden_size=hidden,
               intermediate_size=inter, num_hidden_layers=layers, num_attention_heads=heads,
               num_key_value_heads=kv_heads, head_dim=head_dim, rope_theta=77777.0, rms_norm_eps=7e-6,
               attention_bias=bias, tie_word_embeddings=tied, max_position_embeddings=512)
    if window:
        cfg.update(sliding_window=window,
                   layer_types=["sliding_attention" if i % 2 else "full_attention" for i in range(layers)])
    return cfg


# every head size between the tiny configurations' (16, 24, 64, 128), with widths that no kernel's tile divides
ODD = {"head 32, 7 heads of their own": _odd(136, 40, 2, 7, 7, 32, 331, False, False),
       "head 48, groups of 7, width 100": _odd(100, 172, 2, 14, 2, 48, 1009, True, False),
       "head 80, window 90": _odd(200, 96, 3, 10, 5, 80, 997, False, True, window=90),
       "head 96, window 130": _odd(384, 1000, 2, 12, 4, 96, 4099, False, True, window=130),
       "head 112, groups of 3": _odd(256, 352, 2, 9, 3, 112, 2053, True, True)}


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("shape", list(ODD))
def test_head_sizes_in_steps_of_16(shape, dtype, tmp_path):
    """A batch of unequal prompts and nine single-token steps for head sizes that none of the tiny configurations
    has: the kernels take them, or refuse them; they never answer wrongly."""
    import sleuth_b200 as sb
    cfg = ODD[shape]
    sb.write_random_model(str(tmp_path), cfg, seed=len(shape), dtype=torch.float32)
    eng, ref = load(str(tmp_path), dtype, max_step_tokens=160), oracle(str(tmp_path), dtype)
    rng = np.random.default_rng(len(shape))
    lens = [1, 37, 130, 301, 64]
    reqs = [rng.integers(0, cfg["vocab_size"], size=n + 9).tolist() for n in lens]
    slots = eng.open(len(reqs))
    first = eng.step([(s, r[:n], (n - 1,)) for s, r, n in zip(slots, reqs, lens)]).cpu()
    rows = [[first[i]] for i in range(len(reqs))]
    for k in range(9):
        out = eng.step([(s, [r[n + k]], (0,)) for s, r, n in zip(slots, reqs, lens)]).cpu()
        for i in range(len(reqs)):
            rows[i].append(out[i].clone())
    eng.close(slots)
    eng.stepper.check_status()
    for r, n, got in zip(reqs, lens, rows):
        check(torch.stack(got), ref(r)[n - 1:], TOL[dtype], "engine " + dtype)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("name", ["D", "C", "E"])
def test_chunked_prompt_and_wanted_rows_in_any_order(name, dtype, model_folders):
    """A step longer than max_step_tokens is cut into chunks; wanted places may come in any order. C and E have
    windowed layers (40 and 48 keys): a later chunk of a prompt longer than the window runs after the earlier
    chunks' commit has handed pages back, so its block table starts with entries that hold no page, and its tiles
    begin at different pages."""
    eng = load(model_folders[name], dtype, max_tokens=2048, max_step_tokens=96)
    ref = oracle(model_folders[name], dtype)
    reqs = requests_for(name, [330, 40, 97], seed=3)
    wants = [(329, 0, 95, 96, 191, 192, 63, 64, 287, 288), (), (96, 5)]
    slots = eng.open(3)
    out = eng.step([(s, ids, w) for s, ids, w in zip(slots, reqs, wants)]).cpu()
    if name != "D":
        win = [g for g in eng.cache.book.groups if g.window][0]
        assert win.first_page[slots[0]] >= 4 and (win.table[slots[0]][:4] == -1).all()     # the early pages went back
    eng.close(slots)
    want_rows = torch.stack([ref(ids)[w] for ids, ws in zip(reqs, wants) for w in ws])
    check(out, want_rows, TOL[dtype], "engine " + dtype)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_steps_of_a_repeated_shape_are_recorded_and_still_right(dtype, model_folders):
    """The second step of a shape (tokens, sequences, longest share, wanted rows) is recorded as a CUDA graph and
    replayed from then on. Different tokens, different slots, a different past (a later chunk of a longer prompt)
    and a different split of the same number of tokens between two sequences must each give the plain result."""
    eng, ref = load(model_folders["D"], dtype), oracle(model_folders["D"], dtype)
    reqs = requests_for("D", [150, 150, 150, 300, 150], seed=9)
    seen = 0
    for i, ids in enumerate(reqs[:3]):                     # same shape three times: eager, recorded, replayed
        (slot,) = eng.open(1)
        got = eng.step([(slot, ids, (0, 149))]).cpu()
        check(got, ref(ids)[[0, 149]], TOL[dtype], "engine " + dtype)
        if i == 0:
            held = slot                                     # keep one slot busy so that later ones differ
        else:
            eng.close([slot])
        seen = max(seen, sum(1 for k in eng.stepper._graphs if isinstance(k[0], str)))
    assert seen == 1
    (slot,) = eng.open(1)                                   # the same shape as the second chunk of a longer prompt
    eng.step([(slot, reqs[3][:150], ())])
    got = eng.step([(slot, reqs[3][150:], (0, 149))]).cpu()
    check(got, ref(reqs[3])[[150, 299]], TOL[dtype], "engine " + dtype)
    eng.close([slot, held])
    a, b = requests_for("D", [100, 50], seed=10), requests_for("D", [70, 80], seed=11)
    for pair in (a, b, b[::-1]):                            # 150 tokens in two sequences: shapes (100, ...) and (80, ...)
        slots = eng.open(2)
        got = eng.step([(slots[0], pair[0], (len(pair[0]) - 1,)), (slots[1], pair[1], (len(pair[1]) - 1,))]).cpu()
        check(got, torch.stack([ref(pair[0])[-1], ref(pair[1])[-1]]), TOL[dtype], "engine " + dtype)
        eng.close(slots)


def test_float32_is_bitwise_schedule_independent(model_folders):
    """In float32 every kernel sums in an order that depends on the token's own position only, so a request
    gives the same bits alone, token by token and inside a batch."""
    name = "B"
    eng = load(model_folders[name], "fp32")
    reqs = requests_for(name, [50, 9, 77], seed=1)
    alone = []
    for ids in reqs:
        (s,) = eng.open(1)
        alone.append(eng.step([(s, ids, tuple(range(len(ids))))]).cpu())
        eng.close([s])
    slots = eng.open(3)
    batch = eng.step([(s, ids, tuple(range(len(ids)))) for s, ids in zip(slots, reqs)]).cpu()
    eng.close(slots)
    assert torch.equal(batch, torch.cat(alone))
    (s,) = eng.open(1)
    steps = torch.cat([eng.step([(s, [t], (0,))]).cpu().clone() for t in reqs[1]])
    eng.close([s])
    assert torch.equal(steps, alone[1])


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_through_the_entry_point(name, model_folders):
    import sleuth_b200 as sb
    cfg, w = plain.read_model(model_folders[name])
    eng = load(model_folders[name], "fp32", max_tokens=512)
    prompts = requests_for(name, [3, 12, 30, 1, 8], seed=2)
    want = [plain.greedy_generate(cfg, w, p, 10) for p in prompts]
    res = eng.generate(prompts, max_new_tokens=10, sampling=sb.SamplingConfig(temperature=0.0), stop_ids=(), max_batch=3)
    assert [r.new_ids for r in res] == want and all(r.stop_reason == "max_new_tokens" for r in res)
    one = sb.generate(eng, prompts[1], max_new_tokens=10, sampling=sb.SamplingConfig(temperature=0.0), stop_ids=(),
                      cuda_graph=False)
    assert one.new_ids == want[1] and one.prompt_ids == prompts[1] and one.decode_tok_per_s > 0
    stop = want[2][3]
    res = eng.generate([prompts[2]], max_new_tokens=10, sampling=sb.SamplingConfig(temperature=0.0), stop_ids={stop})
    assert res[0].new_ids == want[2][:want[2].index(stop) + 1] and res[0].stop_reason == "stop_token"
    # bfloat16 follows the same path; its tokens may differ at near-ties, its bookkeeping may not
    eng16 = load(model_folders[name], "bf16", max_tokens=512)
    r16 = eng16.generate(prompts, max_new_tokens=10, sampling=sb.SamplingConfig(temperature=0.0), stop_ids=())
    assert all(len(r.new_ids) == 10 for r in r16)
    # ... and every token it chose must be (within the bfloat16 tolerance) a best token of the plain implementation
    # run on the sequence the engine itself produced: the device-fed loop fed each step the right token
    ref16 = oracle(model_folders[name], "bf16")
    for r in r16:
        rows = ref16(r.prompt_ids + r.new_ids[:-1])[len(r.prompt_ids) - 1:]
        for k, tok in enumerate(r.new_ids):
            assert float(rows[k].max() - rows[k][tok]) <= 2 * TOL["bf16"]["atol"], (name, k, tok)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("name", ["B", "D", "E", "F", "G"])
def test_device_fed_decode_steps_give_the_plain_logits(name, dtype, model_folders):
    """The pipelined loop's steps, driven by hand: the prompt step, the choice left in the device-side feed
    (``choose_later``), then ``decode_fed`` steps that take their tokens from that feed through an index map, with a
    sequence dropping out on the way (so the map is no identity) and the second occurrence of a batch size replayed
    as a graph. The logits of every fed step are compared with the plain implementation for the token the feed held."""
    import sleuth_b200 as sb
    eng, ref = load(model_folders[name], dtype, max_tokens=2048), oracle(model_folders[name], dtype)
    greedy = sb.SamplingConfig(temperature=0.0)
    prompts = requests_for(name, [9, 70, 33, 130], seed=12)
    slots = eng.open(4)
    seqs = [list(p) for p in prompts]
    logits = eng.prefill(slots, prompts)
    check(logits, torch.stack([ref(p)[-1] for p in prompts]), TOL[dtype], "engine " + dtype)
    pending = eng.choose_later(logits, greedy, None, None)
    live = [0, 1, 2, 3]                      # rows of the pending tokens, in feed order
    for step in range(6):
        keep = [i for i in live if not (step == 2 and i == 1)]          # request 1 leaves after two fed steps
        fed = eng.decode_fed([slots[i] for i in keep], [live.index(i) for i in keep])
        nxt = eng.choose_later(fed, greedy, None, None)
        tokens = pending()                                              # the host catches up one step late
        for i, tok in zip(live, tokens):
            seqs[i].append(int(tok))
        check(fed, torch.stack([ref(seqs[i])[-1] for i in keep]), TOL[dtype], "engine " + dtype)
        live, pending = keep, nxt
    eng.close(slots)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("name", ["D", "E"])
def test_a_step_that_mixes_kinds_of_entries(name, dtype, model_folders):
    """One step in which a sequence with 300 tokens behind it brings one token, a fresh sequence brings a 140-token
    prompt, and a third continues by two tokens and wants nothing. The generation loop never builds such a step;
    ``Engine.step`` and the replay program allow it."""
    eng, ref = load(model_folders[name], dtype, max_tokens=2048), oracle(model_folders[name], dtype)
    long, fresh, quiet = requests_for(name, [301, 140, 12], seed=21)
    slots = eng.open(3)
    eng.step([(slots[0], long[:300], ()), (slots[2], quiet[:9], ())])
    out = eng.step([(slots[0], long[300:], (0,)), (slots[1], fresh, (0, 139, 64)), (slots[2], quiet[9:11], ())]).cpu()
    check(out, torch.stack([ref(long)[300], ref(fresh)[0], ref(fresh)[139], ref(fresh)[64]]), TOL[dtype], "engine " + dtype)
    last = eng.step([(slots[2], quiet[11:], (0,)), (slots[1], [5], ())]).cpu()     # what the quiet one appended is there
    check(last, ref(quiet)[11:12], TOL[dtype], "engine " + dtype)
    eng.close(slots)


def test_the_step_tables_may_grow_between_the_choice_and_the_fed_step(model_folders):
    """65 sequences: the single-token step's tables (one more uniform number per sequence) are larger than the prompt
    step's. With a table buffer that holds exactly the prompt step, the first device-fed step replaces the buffer;
    the tokens the sampler left in its feed must survive that."""
    import sleuth_b200 as sb
    from sleuth_b200.engine.batch import MetaStager
    name = "A"
    cfg, w = plain.read_model(model_folders[name])
    eng = load(model_folders[name], "fp32", max_tokens=65 * 64)
    n = 65
    meta = eng.stepper.meta
    _, prompt_total = meta.layout(n, n + 1, n, 0)          # 64 prompts of one token and one of two
    _, decode_total = meta.layout(n, n, n, n)
    assert decode_total > prompt_total
    eng.stepper.meta = MetaStager(eng.device, meta.n_groups, meta.stride, capacity=prompt_total)
    prompts = [[int(t)] for t in np.random.default_rng(3).integers(0, cfg["vocab_size"], size=n)]
    prompts[0] = prompts[0] + [7]
    res = eng.generate(prompts, max_new_tokens=3, sampling=sb.SamplingConfig(temperature=0.7), stop_ids=(), seed=5, max_batch=n)
    assert eng.stepper.meta.generation >= 2 and eng.stepper.meta.cap > prompt_total           # it did grow
    one = load(model_folders[name], "fp32").generate(prompts[:3] + prompts[-2:], max_new_tokens=3,
                                                      sampling=sb.SamplingConfig(temperature=0.7), stop_ids=(), seed=5)
    # request i draws from the stream (seed, i): compare the ones whose index is the same in both runs
    assert [r.new_ids for r in res[:3]] == [r.new_ids for r in one[:3]]
    greedy = eng.generate(prompts, max_new_tokens=3, sampling=sb.SamplingConfig(temperature=0.0), stop_ids=(), max_batch=n)
    for i in (0, 17, 64):
        assert greedy[i].new_ids == plain.greedy_generate(cfg, w, prompts[i], 3)


def test_a_wait_that_runs_out_is_recorded_and_raised():
    """The give-up path of the tensor-memory kernels, run on purpose and harmlessly: a one-block kernel waits a
    thousand polls on a barrier that nothing completes, records its code, frees its tensor memory and returns.
    The host's check must raise, name the code and clear the word; the stepper's late check must do the same."""
    from sleuth_b200.kernels import ops
    ops.gemm_tc_check("cuda:0")                                  # clean before
    ops.tc_wait_probe("cuda:0", polls=1000, code=99)
    torch.cuda.synchronize()
    assert int(ops.tc_status("cuda:0").item()) == 99
    with pytest.raises(RuntimeError, match="code 99"):
        ops.gemm_tc_check("cuda:0")
    ops.gemm_tc_check("cuda:0")                                  # raised once, cleared
    # tensor memory was given back: a product that needs 512 columns of it still runs, and is right
    x = torch.randn(256, 64, device="cuda:0").bfloat16()
    wt = torch.randn(96, 64, device="cuda:0").bfloat16()
    out = torch.empty(256, 96, device="cuda:0", dtype=torch.float32)
    ops.gemm_tc(x, wt, out, "f32")
    torch.testing.assert_close(out, x.float() @ wt.float().T, rtol=1e-3, atol=1e-3)
    ops.gemm_tc_check("cuda:0")


def test_the_stepper_reports_a_given_up_wait_one_step_late(model_folders):
    from sleuth_b200.kernels import ops
    eng = load(model_folders["D"], "bf16")
    ids = requests_for("D", [200], seed=2)[0]
    (slot,) = eng.open(1)
    eng.step([(slot, ids[:150], (149,))])                        # a step of many tokens: the status word is copied after it
    torch.cuda.synchronize()
    ops.tc_wait_probe("cuda:0", polls=1000, code=99)             # ... and something gives up afterwards
    eng.step([(slot, ids[150:190], (0,))])                       # this step's copy sees it
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="code 99"):
        eng.step([(slot, ids[190:191], (0,))])                   # reported when the next step begins
    eng.step([(slot, ids[190:191], (0,))])                       # cleared: the engine goes on
    eng.stepper.check_status()
    eng.close([slot])


def test_context_full_through_the_entry_point(model_folders):
    import sleuth_b200 as sb
    eng = sb.load(model_folders["A"], dtype="fp32", max_seq_len=20, max_tokens=256)
    res = eng.generate([[1, 2, 3] * 6, [4] * 30], max_new_tokens=50, sampling=sb.SamplingConfig(temperature=0.0), stop_ids=())
    assert res[0].stop_reason == "context_full" and len(res[0].new_ids) == 3          # 18 + 2 fed = 20 positions
    assert res[1].prompt_ids == [4] * 19 and res[1].stop_reason == "context_full" and len(res[1].new_ids) == 2


def test_seeded_sampling_is_reproducible_and_batch_independent(model_folders):
    import sleuth_b200 as sb
    eng = load(model_folders["B"], "fp32")
    prompts = requests_for("B", [5, 9, 14], seed=4)
    cfg = sb.SamplingConfig(temperature=0.9, top_k=50, top_p=0.95, min_p=0.01, repetition_penalty=1.2, no_repeat_ngram=3)
    a = eng.generate(prompts, max_new_tokens=12, sampling=cfg, seed=123, stop_ids=())
    b = eng.generate(prompts, max_new_tokens=12, sampling=cfg, seed=123, stop_ids=(), max_batch=1)
    c = eng.generate(prompts, max_new_tokens=12, sampling=cfg, seed=124, stop_ids=())
    assert [r.new_ids for r in a] == [r.new_ids for r in b]
    assert [r.new_ids for r in a] != [r.new_ids for r in c]
    lim = eng.generate(prompts, max_new_tokens=12, sampling=sb.SamplingConfig(temperature=1.5), seed=1, stop_ids=(), vocab_limit=40)
    assert all(t < 40 for r in lim for t in r.new_ids)


@pytest.mark.parametrize("vocab", [503, 151936])
def test_sampler_against_the_plain_pipeline(vocab):
    from sleuth_b200.sampling import SamplingConfig
    from sleuth_b200.sampling.sampler import Sampler
    g = torch.Generator().manual_seed(vocab)
    rows = 6
    logits = torch.randn(rows, vocab, generator=g) * 3
    sampler = Sampler("cuda:0", vocab)
    cases = [SamplingConfig(temperature=0.0), SamplingConfig(temperature=0.7), SamplingConfig(temperature=1.3, top_k=40),
             SamplingConfig(temperature=1.0, top_p=0.8), SamplingConfig(temperature=1.1, min_p=0.05),
             SamplingConfig(temperature=0.9, top_k=200, top_p=0.9, min_p=0.02, repetition_penalty=1.3),
             SamplingConfig(temperature=0.0, repetition_penalty=1.5),
             # more survivors of top-k than the kernel keeps in shared memory: it goes on over the whole row
             SamplingConfig(temperature=0.8, top_k=5000, top_p=0.95), SamplingConfig(temperature=1.2, top_k=3000)]
    recent = [[int(logits[r].argmax()), 3, 7] for r in range(rows)]
    banned = [[int(logits[r].topk(2).indices[1])] if r % 2 else [] for r in range(rows)]
    for ci, cfg in enumerate(cases):
        for trial in range(3):
            u = torch.rand(rows, generator=g).clamp(0, 0.999999)
            got = sampler.to_host(sampler.choose(logits.clone().to("cuda:0"), cfg, u.numpy(), vocab_limit=vocab - 3,
                                                 recent=recent, banned=banned))
            for r in range(rows):
                final = plain.final_logits(logits[r, :vocab - 3], cfg.temperature, cfg.top_k, cfg.top_p, cfg.min_p,
                                           cfg.repetition_penalty, recent[r], banned[r])
                want = int(final.argmax()) if cfg.greedy else plain.draw(final, float(u[r]))
                if got[r] != want:
                    # a draw that lands within rounding of a boundary may pick the neighbour among kept tokens
                    p = final.double().softmax(-1)
                    cdf = p.cumsum(-1)
                    edge = min(abs(float(cdf[want]) - float(u[r])), abs(float(cdf[want] - p[want]) - float(u[r])))
                    assert not cfg.greedy and edge < 1e-5 and float(p[got[r]]) > 0, (ci, trial, r, got[r], want)


def test_sampler_keeps_values_tied_with_the_kth(vocab=40000):
    """Logits on a coarse grid tie by the hundred; top-k keeps every value equal to the k-th (`x < kth` goes), a
    temperature that is no power of two must not split such a tie, and the draw still follows token order."""
    from sleuth_b200.sampling import SamplingConfig
    from sleuth_b200.sampling.sampler import Sampler
    g = torch.Generator().manual_seed(5)
    rows = 4
    logits = (torch.randn(rows, vocab, generator=g) * 3).mul(4).round().div(4)
    sampler = Sampler("cuda:0", vocab)
    for cfg in (SamplingConfig(temperature=0.7, top_k=50), SamplingConfig(temperature=1.3, top_k=3000),
                SamplingConfig(temperature=3.0, top_k=1, min_p=0.0)):
        for trial in range(3):
            u = torch.rand(rows, generator=g).clamp(0, 0.999999)
            got = sampler.to_host(sampler.choose(logits.clone().to("cuda:0"), cfg, u.numpy()))
            for r in range(rows):
                final = plain.final_logits(logits[r], cfg.temperature, cfg.top_k, cfg.top_p, cfg.min_p)
                want = plain.draw(final, float(u[r]))
                if got[r] != want:
                    p = final.double().softmax(-1)
                    cdf = p.cumsum(-1)
                    edge = min(abs(float(cdf[want]) - float(u[r])), abs(float(cdf[want] - p[want]) - float(u[r])))
                    assert edge < 1e-5 and float(p[got[r]]) > 0, (cfg, trial, r, got[r], want)


def test_missing_weights_are_reported_at_load(model_folders, tmp_path):
    import shutil

    import sleuth_b200 as sb
    from sleuth_b200.weights import WeightError, read_safetensors, write_safetensors
    d = tmp_path / "broken"
    shutil.copytree(model_folders["A"], d)
    t = read_safetensors(d / "model.safetensors")
    del t["model.layers.0.mlp.gate_proj.weight"]
    write_safetensors(t, d / "model.safetensors")
    with pytest.raises(WeightError, match="missing.*gate_proj"):
        sb.load(d, dtype="fp32")


@pytest.mark.parametrize("rows", ["tensor-memory kernel for every product", "weight-streaming kernel up to 64 rows"])
def test_bfloat16_engine_on_each_own_product_kernel(rows, model_folders, monkeypatch):
    """The engine picks its product kernel by row count; here each own kernel is made to serve every product it
    can take, prompts and single tokens alike, and the logits must still match the plain implementation."""
    from sleuth_b200.parts import linear
    if rows.startswith("tensor"):
        monkeypatch.setattr(linear, "SKINNY_ROWS", 0)
        monkeypatch.setattr(linear, "TC_ROWS", 1)
    else:
        monkeypatch.setattr(linear, "SKINNY_ROWS", 64)
    monkeypatch.setenv("SLEUTH_B200_CHECK", "1")
    for name in ("C", "D"):
        eng, ref = load(model_folders[name], "bf16", use_graphs=False), oracle(model_folders[name], "bf16")
        reqs = requests_for(name, [150, 40, 9], seed=6)
        slots = eng.open(3)
        out = eng.step([(s, ids[:-1], (len(ids) - 2,)) for s, ids in zip(slots, reqs)]).cpu()
        check(out, torch.stack([ref(ids)[-2] for ids in reqs]), TOL["bf16"], "engine " + "bf16")
        out = eng.step([(s, ids[-1:], (0,)) for s, ids in zip(slots, reqs)]).cpu()
        check(out, torch.stack([ref(ids)[-1] for ids in reqs]), TOL["bf16"], "engine " + "bf16")
        eng.close(slots)
        from sleuth_b200.kernels import ops
        ops.gemm_tc_check("cuda:0")


@pytest.mark.parametrize("name", ["F", "G"])
def test_persistent_single_token_kernel(name, model_folders, monkeypatch):
    """SLEUTH_B200_DECODE=fused: single-token steps of up to 16 sequences run all layers in one persistent kernel
    (csrc/decode_layers.cu) where the sizes allow it, as F's and G's do. Prefix then the last 32 tokens one by one
    (several pages, F's windowed layer, the step replayed as a graph), unequal batches that end early and whose
    slots and pages are used again, steps fed from the device: all against the plain implementation."""
    import sleuth_b200 as sb
    from sleuth_b200.engine import model as model_mod
    monkeypatch.setattr(model_mod, "DECODE_CHOICE", "fused")
    dtype = "bf16"
    eng, ref = load(model_folders[name], dtype, max_tokens=64 * 12), oracle(model_folders[name], dtype)
    assert eng.model._fused_runs(type("B", (), dict(max_count=1, T=3, n=3))(), eng.cache)      # the sizes qualify
    for ids in requests_for(name, [300, 70], seed=31):
        cut = len(ids) - 32
        (slot,) = eng.open(1)
        rows = [eng.step([(slot, ids[:cut], (cut - 1,))]).cpu()]
        for t in ids[cut:]:
            rows.append(eng.step([(slot, [t], (0,))]).cpu().clone())
        eng.close([slot])
        check(torch.cat(rows), ref(ids)[cut - 1:], TOL[dtype], "engine " + dtype)
    plans = [[(100, 20), (60, 3), (5, 27), (130, 9)], [(1, 12), (64, 1), (63, 2), (30, 30), (200, 5)]]
    for b, plan in enumerate(plans):
        reqs = requests_for(name, [p + d for p, d in plan], seed=40 + b)
        slots = eng.open(len(reqs))
        got = {i: [] for i in range(len(reqs))}
        out = eng.step([(s, ids[:p], (p - 1,)) for s, ids, (p, d) in zip(slots, reqs, plan)]).cpu()
        for i in range(len(reqs)):
            got[i].append(out[i])
        live, k = list(range(len(reqs))), 0
        while live:
            out = eng.step([(slots[i], [reqs[i][plan[i][0] + k]], (0,)) for i in live]).cpu()
            for j, i in enumerate(live):
                got[i].append(out[j].clone())
            done = [i for i in live if k + 1 >= plan[i][1]]
            eng.close([slots[i] for i in done])
            live = [i for i in live if i not in done]
            k += 1
        for i, ids in enumerate(reqs):
            check(torch.stack(got[i]), ref(ids)[plan[i][0] - 1:], TOL[dtype], "engine " + dtype)
    assert eng.cache.book.pages_in_use() == [0] * eng.cache.n_groups
    res = eng.generate(requests_for(name, [9, 70, 33], seed=50), max_new_tokens=6, sampling=sb.SamplingConfig(temperature=0.0), stop_ids=())
    for r in res:                                   # the device-fed loop through the same kernel
        rows = ref(r.prompt_ids + r.new_ids[:-1])[len(r.prompt_ids) - 1:]
        for k, tok in enumerate(r.new_ids):
            assert float(rows[k].max() - rows[k][tok]) <= 2 * TOL[dtype]["atol"], (name, k, tok)
    eng.stepper.check_status()
