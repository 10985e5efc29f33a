"""Host-side mirror of the reference interface: op schemas, wrappers, helpers,
workload generators (no GPU needed)."""
import inspect

import numpy as np
import pytest
import torch

from vllm_b200 import _custom_ops as ops
import workloads as W
from vllm_b200.paged_attn import PagedAttention, _PARTITION_SIZE


def _norm(s):
    return "".join(str(s).split())


def test_schemas_equal_the_reference_declarations():
    ops.claim_reference_names()
    # csrc/torch_bindings.cpp:52-76, :687-704, :716-719 of the reference
    want_v1 = ("paged_attention_v1(Tensor! out, Tensor query, Tensor key_cache, Tensor value_cache, "
               "int num_kv_heads, float scale, Tensor block_tables, Tensor seq_lens, int block_size, "
               "int max_seq_len, Tensor? alibi_slopes, str kv_cache_dtype, Tensor k_scale, Tensor v_scale, "
               "int tp_rank, int blocksparse_local_blocks, int blocksparse_vert_stride, "
               "int blocksparse_block_size, int blocksparse_head_sliding_step) -> ()")
    for ns in ("_C", "_C_b200"):
        got = getattr(torch.ops, ns).paged_attention_v1.default._schema
        assert _norm(got) == _norm(torch._C.parse_schema(f"{ns}::" + want_v1))
    v2 = torch.ops._C.paged_attention_v2.default._schema
    names = [a.name for a in v2.arguments]
    assert names[:5] == ["out", "exp_sums", "max_logits", "tmp_out", "query"]
    assert [a.alias_info is not None and a.alias_info.is_write for a in v2.arguments[:5]] == [True] * 4 + [False]
    for name in ("reshape_and_cache", "reshape_and_cache_flash"):
        sch = getattr(torch.ops._C_cache_ops, name).default._schema
        assert [a.name for a in sch.arguments] == ["key", "value", "key_cache", "value_cache",
                                                    "slot_mapping", "kv_cache_dtype", "k_scale", "v_scale"]
        writes = [a.alias_info is not None and a.alias_info.is_write for a in sch.arguments]
        assert writes == [False, False, True, True, False, False, False, False]
        assert len(sch.returns) == 0
    cf = torch.ops._C_cache_ops.convert_fp8.default._schema
    assert [a.name for a in cf.arguments] == ["dst_cache", "src_cache", "scale", "kv_cache_dtype"]


def test_wrapper_signatures_match_reference_wrappers():
    # vllm/_custom_ops.py:29-48, :73-95 of the reference
    p = list(inspect.signature(ops.paged_attention_v1).parameters)
    assert p == ["out", "query", "key_cache", "value_cache", "num_kv_heads", "scale", "block_tables",
                 "seq_lens", "block_size", "max_seq_len", "alibi_slopes", "kv_cache_dtype", "k_scale",
                 "v_scale", "tp_rank", "blocksparse_local_blocks", "blocksparse_vert_stride",
                 "blocksparse_block_size", "blocksparse_head_sliding_step"]
    p2 = list(inspect.signature(ops.paged_attention_v2).parameters)
    assert p2 == ["out", "exp_sum", "max_logits", "tmp_out"] + p[1:]
    d = inspect.signature(ops.paged_attention_v1).parameters
    assert d["blocksparse_block_size"].default == 64 and d["tp_rank"].default == 0


def test_ops_are_cuda_only_like_the_reference():
    q = torch.zeros(2, 4, 128, dtype=torch.bfloat16)
    kc = torch.zeros(4, 2, 16, 16, 8, dtype=torch.bfloat16)
    vc = torch.zeros(4, 2, 128, 16, dtype=torch.bfloat16)
    bt = torch.zeros(2, 2, dtype=torch.int32)
    sl = torch.ones(2, dtype=torch.int32)
    one = torch.tensor(1.0)
    with pytest.raises((RuntimeError, NotImplementedError)):
        ops.paged_attention_v1(torch.empty_like(q), q, kc, vc, 2, 0.1, bt, sl, 16, 16, None, "auto", one, one)
    with pytest.raises((RuntimeError, NotImplementedError)):
        ops.reshape_and_cache(q, q, kc, vc, torch.zeros(2, dtype=torch.int64), "auto", one, one)


def test_paged_attention_helper_shapes_and_split():
    assert PagedAttention.get_supported_head_sizes() == [32, 64, 80, 96, 112, 120, 128, 192, 256]
    assert _PARTITION_SIZE == 512
    shape = PagedAttention.get_kv_cache_shape(10, 16, 8, 128)
    assert shape == (2, 10, 16 * 8 * 128)
    kv = torch.zeros(shape, dtype=torch.bfloat16)
    k, v = PagedAttention.split_kv_cache(kv, 8, 128)
    assert k.shape == (10, 8, 16, 16, 8) and v.shape == (10, 8, 128, 16)
    kv8 = torch.zeros(shape, dtype=torch.uint8)
    k8, v8 = PagedAttention.split_kv_cache(kv8, 8, 128)
    assert k8.shape == (10, 8, 8, 16, 16) and v8.shape == (10, 8, 128, 16)
    assert k.data_ptr() == kv.data_ptr() and v.data_ptr() == kv[1].data_ptr()


def test_workload_generators_are_deterministic_and_well_formed():
    a = W.small("cpu", seed=3)
    b = W.small("cpu", seed=3)
    assert torch.equal(a.query, b.query) and torch.equal(a.block_tables, b.block_tables)
    assert torch.equal(a.key_cache, b.key_cache)
    lens = a.seq_lens.numpy()
    need = np.ceil(lens / a.block_size).astype(int)
    for s in range(a.num_seqs):
        row = a.block_tables[s, :need[s]].numpy()
        assert len(set(row.tolist())) == len(row)          # sample without replacement
        assert (a.block_tables[s, need[s]:] == 0).all()     # zero padded
    by = a.attn_bytes()
    kv = int(lens.sum()) * a.num_kv_heads * a.head_size * 2 * 2
    qo = 2 * a.num_seqs * a.num_heads * a.head_size * 2
    assert by == kv + qo + 4 * int(need.sum()) + 4 * a.num_seqs


def test_config_plans_match_the_stated_shapes():
    rng = np.random.default_rng(0)
    lens2 = rng.integers(512, 4097, size=256)
    assert lens2.min() >= 512 and lens2.max() <= 4096
    rng = np.random.default_rng(0)
    lens4 = np.clip(np.round(rng.lognormal(8.5, 1.0, size=64)), 16, 32768)
    assert lens4.min() >= 16 and lens4.max() <= 32768
    w = W.make_decode("t", num_seqs=3, num_heads=8, num_kv_heads=1, head_size=128, block_size=32,
                      lens=np.array([5, 70, 33]), dtype=torch.bfloat16, kv_cache_dtype="fp8",
                      device="cpu", seed=0, rng=np.random.default_rng(0))
    assert w.key_cache.dtype == torch.uint8 and w.key_cache.shape[2:] == (8, 32, 16)
    assert w.value_cache.shape[1:] == (1, 128, 32)
    tot = int(np.ceil(np.array([5, 70, 33]) / 32).sum())
    used = set()
    for s, n in enumerate([1, 3, 2]):
        used |= set(w.block_tables[s, :n].tolist())
    assert len(used) == tot                                  # globally unique blocks
    assert w.key_cache.shape[0] == int(np.ceil(1.25 * tot))


def test_token_ranges_cover_every_token_once_at_block_boundaries():
    """Token sharding plan (decode context parallelism): the ranks' ranges of a sequence are
    block-aligned, contiguous, disjoint and together cover it; the ragged tail goes to one rank."""
    import numpy as np
    import workloads as W

    lens = np.array([0, 1, 15, 16, 17, 700, 4096, 4097, 33])
    for block_size in (16, 32):
        for world in (1, 2, 3, 8):
            total = np.zeros_like(lens)
            prev_end = np.zeros_like(lens)
            for rank in range(world):
                b0, b1, toks = W.token_ranges(lens, block_size, world, rank)
                assert np.all(b0 == prev_end) and np.all(b1 >= b0)
                full = (b1 - b0) * block_size
                assert np.all(toks <= full) and np.all(toks >= 0)
                # only the range that ends the sequence may be ragged
                ragged = toks < full
                assert np.all(b1[ragged] * block_size >= lens[ragged])
                total += toks
                prev_end = b1
            assert np.array_equal(total, lens)
            assert np.array_equal(prev_end, (lens + block_size - 1) // block_size)


def test_reference_names_are_claimed_on_request_and_never_twice():
    """Loading the package defines torch.ops._C_b200.* only.  The reference's own names are
    registered by an explicit call (so that a vLLM extension imported later can still define
    them itself), once: a second call finds them taken and claims nothing."""
    import subprocess
    import sys
    code = (
        "import torch\n"
        "from vllm_b200 import _custom_ops as ops\n"
        "has = lambda: hasattr(torch.ops._C, 'paged_attention_v1') and hasattr(torch.ops._C_cache_ops, 'reshape_and_cache')\n"
        "a = has()\n"
        "n1 = ops.claim_reference_names()\n"
        "b = has()\n"
        "n2 = ops.claim_reference_names()\n"
        "print(a, n1, b, n2)\n")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True,
                       cwd=str(__import__("pathlib").Path(__file__).resolve().parents[1]))
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.split() == ["False", "8", "True", "0"]


def test_moved_tiles_of_the_kv_write_cover_every_token():
    """The staged KV write may move a 16-token tile onto the next 16-slot boundary of the cache
    (vllm_b200/csrc/kv_write_staged.cuh, `shift_of`): tile i then covers tokens
    [16 i + s_i, 16 i + s_i + 16) and writes the tokens [16 i + s_(i-1), 16 i + s_i) in front of
    its window itself when the tile before it is moved by less.  Whatever the slots are, every
    token must be covered at least once.  This restates the rule on the host and checks the
    property on random slot mappings (runs of consecutive slots at odd offsets, scattered tokens,
    padding)."""
    import numpy as np

    def shift_of(first, mid, last):
        if first < 0 or mid < 0 or last < 0:
            return 0
        if (mid - first) % 16 != 8 or (last - first) % 16 != 15:
            return 0
        return (16 - first % 16) % 16

    def tile_shift(slots, i):
        T = len(slots)
        tok = [16 * i, 16 * i + 8, 16 * i + 15]
        if i < 0 or tok[2] >= T:
            return 0
        return shift_of(*(int(slots[t]) for t in tok))

    rng = np.random.default_rng(5)
    for _ in range(300):
        pieces, free = [], 0
        for _ in range(int(rng.integers(1, 30))):
            kind = int(rng.integers(4))
            if kind == 0:
                free += int(rng.integers(1, 80))
                pieces.append(np.array([free]))
                free += 1
            elif kind == 1:
                pieces.append(np.full(int(rng.integers(1, 9)), -1))
            else:
                n = int(rng.integers(1, 90))
                free += int(rng.integers(0, 48))
                pieces.append(np.arange(free, free + n))
                free += n
        order = rng.permutation(len(pieces))
        slots = np.concatenate([pieces[k] for k in order])
        T = len(slots)
        covered = np.zeros(T, dtype=int)
        for i in range((T + 15) // 16):
            s, sp = tile_shift(slots, i), tile_shift(slots, i - 1)
            covered[16 * i + s:min(16 * i + s + 16, T)] += 1          # the window
            if s > 0:
                covered[16 * i + (sp if i > 0 else 0):min(16 * i + s, T)] += 1  # the tokens in front
        assert (covered >= 1).all(), (slots.tolist(), covered.tolist())
