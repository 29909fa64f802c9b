"""Host-side behaviour that needs no GPU: the module's API surface, error behaviour,
and the sharding arithmetic."""
import pytest
import torch


def test_module_surface_matches_reference(pkg):
    m = pkg.FusedGatedMLP()  # reference defaults: hidden 256, intermediate 512, bias, silu, p=0
    assert (m.hidden_size, m.intermediate_size, m.act_fn, m.dropout.p) == (256, 512, "silu", 0.0)
    names = [n for n, _ in m.named_parameters()]
    assert names == ["gate_proj.weight", "gate_proj.bias", "up_proj.weight", "up_proj.bias",
                     "down_proj.weight", "down_proj.bias"]
    assert m.gate_proj.weight.shape == (512, 256) and m.down_proj.weight.shape == (256, 512)
    m2 = pkg.FusedGatedMLP(64, 128, bias=False, dropout_p=0.25)
    assert m2.gate_proj.bias is None and m2.dropout.p == 0.25
    # state_dict round trip with a plain torch twin (what copy_weights of the reference relies on)
    twin = torch.nn.ModuleDict({"gate_proj": torch.nn.Linear(256, 512), "up_proj": torch.nn.Linear(256, 512),
                                "down_proj": torch.nn.Linear(512, 256)})
    m.load_state_dict(twin.state_dict())
    assert torch.equal(m.up_proj.weight, twin["up_proj"].weight)


def test_unsupported_activation_and_modes(pkg):
    with pytest.raises(NotImplementedError):
        pkg.FusedGatedMLP(hidden_act="mish")
    for name in ("gelu", "relu", "sigmoid", "tanh", "leaky_relu", "no_act", "swish"):
        m = pkg.FusedGatedMLP(64, 128, hidden_act=name)
        assert m.act_fn == name and isinstance(m.act, torch.nn.Module)
    with pytest.raises(ValueError):
        pkg.FusedGatedMLP(parallel_mode="pipeline")


def test_no_cpu_fallback(pkg):
    m = pkg.FusedGatedMLP(64, 128).to(torch.bfloat16)
    with pytest.raises(pkg._lib.GmlpError, match="no CPU path"):
        m(torch.zeros(4, 64, dtype=torch.bfloat16))


def test_op_level_preconditions(pkg):
    x = torch.zeros(4, 64)
    w = torch.zeros(128, 64)
    with pytest.raises(AssertionError):
        pkg.mlp_hidden_states_fwd(torch.zeros(2, 4, 64), w, None, w, None, "silu", 0.0)
    with pytest.raises(AssertionError):
        pkg.mlp_hidden_states_fwd(x, torch.zeros(128, 32), None, w, None, "silu", 0.0)
    with pytest.raises(AssertionError):
        pkg.mlp_hidden_states_fwd(x, w, torch.zeros(64), w, None, "silu", 0.0)
    with pytest.raises(NotImplementedError):
        pkg.mlp_hidden_states_fwd(torch.zeros(4, 24), torch.zeros(128, 24), None, torch.zeros(128, 24), None,
                                  "silu", 0.0)
    with pytest.raises(NotImplementedError):
        pkg.mlp_hidden_states_fwd(x, w, None, w, None, "softplus", 0.0)


def test_dtype_code(pkg):
    assert pkg._lib.dtype_code(torch.bfloat16) == 0 and pkg._lib.dtype_code(torch.float16) == 1
    assert pkg._lib.dtype_code(torch.float32) == 2      # fp32 matrices, tf32 products
    with pytest.raises(NotImplementedError):
        pkg._lib.dtype_code(torch.float64)


def test_token_shard_ranges_cover_rows_once(pkg):
    P = pkg.parallel
    for m, w in ((8192, 8), (65536, 4), (10, 4), (3, 8)):
        spans = [P.token_shard_range(m, r, w) for r in range(w)]
        assert spans[0][0] == 0 and sum(c for _, c in spans) == m
        assert all(spans[i][0] + spans[i][1] == spans[i + 1][0] for i in range(w - 1))
    with pytest.raises(ValueError):
        P.token_shard_range(8, 8, 8)


def test_tp_shard_ranges_and_state_dict(pkg):
    P = pkg.parallel
    assert P.tp_shard_range(28672, 3, 8) == (3 * 3584, 3584)
    with pytest.raises(ValueError):
        P.tp_shard_range(28672 + 16, 0, 8)
    full = {
        "gate_proj.weight": torch.arange(64.0 * 8).reshape(64, 8), "gate_proj.bias": torch.arange(64.0),
        "up_proj.weight": -torch.arange(64.0 * 8).reshape(64, 8), "up_proj.bias": -torch.arange(64.0),
        "down_proj.weight": torch.arange(8.0 * 64).reshape(8, 64), "down_proj.bias": torch.arange(8.0),
    }
    parts = [P.shard_tp_state_dict(full, r, 2) for r in range(2)]
    assert torch.equal(torch.cat([p["gate_proj.weight"] for p in parts]), full["gate_proj.weight"])
    assert torch.equal(torch.cat([p["down_proj.weight"] for p in parts], dim=1), full["down_proj.weight"])
    assert torch.equal(parts[1]["up_proj.bias"], full["up_proj.bias"][32:])
    assert torch.equal(parts[1]["down_proj.bias"], full["down_proj.bias"])


def test_module_shard_descriptor(pkg):
    m = pkg.FusedGatedMLP(64, 128, parallel_mode="tp", tp_rank=2, tp_size=4)
    s = m._shard()
    assert (s.row0, s.col0, s.n_global) == (0, 256, 512)
    t = pkg.FusedGatedMLP(64, 128, parallel_mode="token")
    t.token_row0 = 4096
    assert (t._shard().row0, t._shard().col0) == (4096, 0)


def test_tuning_travels_with_the_call_not_with_the_process(pkg):
    """GEMM tuning is a field of each call's problem descriptor. Switching one module's SM limit on must not
    move the process-wide defaults that every other module, device and host thread reads."""
    L = pkg._lib
    lib = L.load()
    assert L.tune_word() == 0
    w = L.tune_word(pair_mode=2, raster_group=16, sm_limit=132)
    assert (w & 3, (w >> 2) & 0xFFF, (w >> 14) & 0xFFF) == (2, 16, 132)
    assert L.tune_word(ordinary_launch=True) == 1 << 26 and L.tune_word(sm_limit=4095) < 1 << 26
    assert L.tune_word(narrow_tiles=True) == 1 << 27
    with pytest.raises(ValueError):
        L.tune_word(sm_limit=5000)
    from triton_gated_mlp_b200.gated_mlp import _SmLimit

    before = (lib.gmlp_set_cta_pair_mode(-1), lib.gmlp_set_raster_group(-1), lib.gmlp_set_sm_limit(-1))  # queries
    lim = _SmLimit(torch.device("cpu"), 16, sm_count=148)
    assert lim.tuning == 0
    lim(True)
    assert lim.tuning == L.tune_word(sm_limit=132)
    assert (lib.gmlp_set_cta_pair_mode(-1), lib.gmlp_set_raster_group(-1), lib.gmlp_set_sm_limit(-1)) == before
    lim(False)
    assert lim.tuning == 0
    # the descriptor carries the word
    p = pkg.ops.kernels._problem(4, 64, 64, torch.bfloat16, pkg.ops.kernels.NO_DROPOUT, pkg.ops.kernels.NO_SHARD,
                                 tuning=w)
    assert p.tuning == w


def test_status_read_moves_the_scratch_epoch_only_on_failure(pkg):
    L = pkg._lib
    e0 = L.scratch_epoch()
    assert isinstance(e0, int) and L.scratch_epoch() == e0
