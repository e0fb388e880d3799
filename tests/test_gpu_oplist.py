"""The op-list mode (MLP / GPT-2 shaped models, base-field challenges, ops proved in reverse on one
transcript) on the GPU against the oracle's restatement of pipeline/forward.rs + pipeline/prove.rs:
bincode(Vec<SerializedLayerProof>) must be identical byte for byte."""
import numpy as np
import pytest

import zklm_compile_b200 as zk
from zklm_compile_b200 import oplist as zo, tables
from oracle import pyoracle as O

pytestmark = pytest.mark.gpu
P = (1 << 31) - 1


@pytest.fixture(scope="module")
def env():
    c = zk.Context(0)
    gelu = tables.build_gelu_table(1000)
    yield c, gelu, c.upload(gelu)
    c.close()


def _w(rng, n):
    return np.mod(rng.integers(-127, 128, n), P).astype(np.uint32)


class Pair:
    """Builds the same op list on the GPU and in the oracle.  Ops whose data the reference gets from
    its Python driver (the requantised gelu pairs, the set_input values) are computed by the oracle
    side from its own forward pass; the GPU computes them on the device."""

    def __init__(self, ctx, x):
        self.g, self.o, self.x = zo.OpList(ctx, len(x)), O.OpList(), x

    def linear(self, name, w, b, m, n):
        self.g.linear(name, w, b, m, n); self.o.linear(name, w, b, m, n)

    def relu(self, name):
        self.g.relu(name); self.o.simple("relu", name)

    def layernorm(self, name, gamma, beta):
        self.g.layernorm(name, gamma, beta); self.o.layernorm(name, gamma, beta)

    def attention(self, name):
        self.g.attention_seq1(name); self.o.simple("attention", name)

    def save(self, name, key):
        self.g.save(name, key); self.o.simple("save", name, key)

    def add_saved(self, name, key):
        self.g.add_saved(name, key); self.o.simple("add_saved", name, key)

    def passthrough(self, name):
        self.g.passthrough(name); self.o.simple("passthrough", name)

    def gelu(self, name, table_host, table_dev):
        cur = self.o.forward(self.x)
        q = O.requantize(cur)
        idx = np.where(q.astype(np.int64) > P // 2, q.astype(np.int64) - P + len(table_host), q.astype(np.int64))
        self.g.gelu(name, table_dev); self.o.gelu(name, q, table_host[idx], table_host)

    def set_input_requant(self, name):
        cur = self.o.forward(self.x)
        self.g.set_input_requant(name); self.o.set_input(name, O.requantize(cur))

    def check(self):
        exp = self.o.prove(self.x)
        got = self.g.prove(self.x)
        assert self.g.activation().tolist() == self.o.forward(self.x).tolist(), "forward output differs"
        assert len(got) == len(exp) and got == exp, "op-list proof bytes differ from the oracle"
        assert self.g.prove(self.x) == exp                     # and again on the same resident list
        self.g.close()
        return got


def test_mlp_with_relu_matches_oracle(env):
    """The published Dense-4M structure (linear, relu, linear, relu, linear) at 1/16 scale; the second
    relu is proved right after a matmul, so its chain-evaluation proof is exercised."""
    c = env[0]
    rng = np.random.default_rng(1)
    dims = [64, 128, 64, 10]
    x = _w(rng, dims[0])
    p = Pair(c, x)
    for l in range(3):
        p.linear(f"fc{l}", _w(rng, dims[l + 1] * dims[l]), _w(rng, dims[l + 1]), dims[l + 1], dims[l])
        if l < 2:
            p.relu(f"relu{l}")
    proof = p.check()
    assert int.from_bytes(proof[:8], "little") == 5


def test_layernorm_alone_and_perturbed(env):
    """LayerNormSqr for several widths (a non-power-of-two pads) and seeds; with 200 candidate inputs
    about half need the QR perturbation of x[0]."""
    c = env[0]
    for seed, d in [(2, 48), (3, 64), (4, 100), (5, 768)]:
        rng = np.random.default_rng(seed)
        x = _w(rng, d)
        p = Pair(c, x)
        p.layernorm("ln", _w(rng, d), _w(rng, d))
        p.check()


def test_gpt2_block_ops_match_oracle(env):
    """One GPT-2-shaped block at small width with every op kind of the reference's GPT-2 op list:
    save, layernorm, c_attn, attention (seq_len 1), c_proj, add_saved, set_input, save, layernorm,
    mlp_fc, gelu, set_input, mlp_proj, add_saved, set_input, final layernorm, lm_head."""
    c, gelu_h, gelu_d = env
    rng = np.random.default_rng(7)
    D, F, V = 48, 160, 301
    x = _w(rng, D)
    p = Pair(c, x)
    p.save("save_res1_0", "res1_0")
    p.layernorm("ln1_0", _w(rng, D), _w(rng, D))
    p.linear("c_attn_0", _w(rng, 3 * D * D), _w(rng, 3 * D), 3 * D, D)
    p.attention("attn_0")
    p.linear("c_proj_0", _w(rng, D * D), _w(rng, D), D, D)
    p.add_saved("add_res1_0", "res1_0")
    p.set_input_requant("in_mlp_fc_0")
    p.save("save_res2_0", "res2_0")
    p.layernorm("ln2_0", _w(rng, D), _w(rng, D))
    p.linear("mlp_fc_0", _w(rng, F * D), _w(rng, F), F, D)
    p.gelu("gelu_0", gelu_h, gelu_d)
    p.set_input_requant("in_mlp_proj_0")
    p.linear("mlp_proj_0", _w(rng, D * F), _w(rng, D), D, F)
    p.add_saved("add_res2_0", "res2_0")
    p.set_input_requant("in_lm_head")
    p.layernorm("final_ln", _w(rng, D), _w(rng, D))
    p.linear("lm_head", _w(rng, V * D), None, V, D)
    p.passthrough("tail")
    proof = p.check()
    assert int.from_bytes(proof[:8], "little") == 18


def test_set_input_first_op_and_explicit_values(env):
    """set_input as the very first op hashes 32 zero bytes for the missing previous output
    (prove.rs:462-470); explicit values are taken as they are."""
    c = env[0]
    rng = np.random.default_rng(9)
    x = _w(rng, 16)
    v = _w(rng, 32)
    g, o = zo.OpList(c, 16), O.OpList()
    g.set_input("in0", v); o.set_input("in0", v)
    w = _w(rng, 8 * 32)
    g.linear("fc", w, None, 8, 32); o.linear("fc", w, None, 8, 32)
    assert g.prove(x) == o.prove(x)
    g.close()


def test_op_list_argument_errors(env):
    c = env[0]
    rng = np.random.default_rng(1)
    g = zo.OpList(c, 16)
    with pytest.raises(zk.ZkbError) as e:
        g.linear("bad", _w(rng, 8 * 15), None, 8, 15)          # column count != activation length
    assert e.value.code == 6
    with pytest.raises(zk.ZkbError):
        g.add_saved("add_x", "never_saved")
    with pytest.raises(zk.ZkbError):
        g.attention_seq1("attn")                               # 16 is not a multiple of 3
    # a failed add leaves the list as it was: it still takes ops of the old activation length and proves
    x = _w(rng, 16)
    w = _w(rng, 4 * 16)
    g.linear("fc", w, None, 4, 16)
    o = O.OpList()
    o.linear("fc", w, None, 4, 16)
    assert g.prove(x) == o.prove(x)
    g.close()
