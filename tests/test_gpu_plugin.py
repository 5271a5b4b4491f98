"""The plugin surface end to end on a GPU: SparsityBuilder -> F.linear / torch.mm dispatch -> backward, pickling,
device moves.  Numerical reference is torch on the densified weight (fp32 tolerance 1e-5 relative Frobenius)."""
import io
import warnings

import numpy as np
import pytest
import torch

from gpu_util import cuda, np_of, rel_fro, seeded_normal

pytestmark = pytest.mark.gpu


class FFN(torch.nn.Module):
    def __init__(self, d=768, h=3072):
        super().__init__()
        self.fc1 = torch.nn.Linear(d, h)
        self.act = torch.nn.GELU()
        self.fc2 = torch.nn.Linear(h, d)

    def forward(self, x):
        return self.fc2(self.act(self.fc1(x)))


def _sparsify(model, n, m, g):
    import sten_b200 as sten
    sb = sten.SparsityBuilder()
    for name, mod in model.named_modules():
        if isinstance(mod, torch.nn.Linear):
            sb.set_weight(name=name + ".weight", initial_sparsifier=sten.GroupedNMSparsifier(n=n, m=m, g=g),
                          out_format=sten.GroupedNMTensor)
    return sb.get_sparse_model(model)


def _densified_copy(sparse_model, template):
    import copy
    import sten_b200 as sten
    dense = copy.deepcopy(template)
    for (name, p), (_, q) in zip(sparse_model.named_parameters(), dense.named_parameters()):
        src = p.wrapped_tensor.to_dense() if isinstance(p, sten.SparseTensorWrapper) else p
        q.data.copy_(src.detach())
    return dense


def test_ffn_pair_forward_and_dx_backward_bert_base_shapes():
    """BERT-base FFN pair at 1:4, linear -> GELU -> linear, forward plus the dX pass."""
    import sten_b200 as sten
    torch.manual_seed(0)
    model = FFN().to(cuda())
    sparse = _sparsify(model, 1, 4, 16)
    assert isinstance(sparse.fc1.weight, sten.SparseParameterWrapper)
    dense = _densified_copy(sparse, model).double()
    x = seeded_normal((8, 512, 768), 1).to(cuda()).requires_grad_(True)
    sten.set_dispatch_failure("raise")  # any fall-back to dense would raise: the CUDA kernels must be the path
    y = sparse(x)
    xd = x.detach().double().requires_grad_(True)
    yd = dense(xd)
    assert rel_fro(np_of(y), yd.detach().cpu().numpy()) <= 1e-5
    dy = seeded_normal((8, 512, 768), 2).to(cuda())
    for p in sparse.parameters():
        p.requires_grad_(False)
    y.backward(dy)
    yd.backward(dy.double())
    assert rel_fro(np_of(x.grad), xd.grad.cpu().numpy()) <= 1e-5


def test_bias_free_linear_uses_the_kernel_and_mm_dispatch():
    import sten_b200 as sten
    sten.set_dispatch_failure("raise")
    lin = torch.nn.Linear(200, 64, bias=False).to(cuda())
    sparse = _sparsify(torch.nn.Sequential(lin), 2, 4, 8)
    x = seeded_normal((50, 200), 3).to(cuda())
    w = sparse[0].weight
    with warnings.catch_warnings():
        warnings.simplefilter("error", sten.DispatchWarning)
        y = sparse(x)
        wd = w.wrapped_tensor.to_dense()
        assert rel_fro(np_of(y), np_of(x).astype(np.float64) @ np_of(wd).astype(np.float64).T) <= 1e-5
        b = seeded_normal((200, 33), 4).to(cuda()).requires_grad_(True)
        c = torch.mm(w, b)
        assert rel_fro(np_of(c), np_of(wd).astype(np.float64) @ np_of(b).astype(np.float64)) <= 1e-5
        c.sum().backward()
        want = np_of(wd).astype(np.float64).T @ np.ones((64, 33))
        assert rel_fro(np_of(b.grad), want) <= 1e-5


def test_trainable_weight_gets_dense_gradient_wrapper():
    import sten_b200 as sten
    lin = torch.nn.Linear(96, 32).to(cuda())
    sparse = _sparsify(torch.nn.Sequential(lin), 2, 4, 4)
    x = seeded_normal((10, 96), 6).to(cuda())
    sparse(x).sum().backward()
    g = sparse[0].weight.grad
    assert isinstance(g, sten.SparseTensorWrapper) and isinstance(g.wrapped_tensor, sten.DenseTensor)
    assert rel_fro(np_of(g.wrapped_tensor.to_dense()), np.ones((32, 10)) @ np_of(x).astype(np.float64)) <= 1e-5


def test_pickle_round_trip_and_device_move():
    import sten_b200 as sten
    lin = torch.nn.Linear(120, 48).to(cuda())
    sparse = _sparsify(torch.nn.Sequential(lin), 2, 8, 2)
    x = seeded_normal((7, 120), 8).to(cuda())
    y = sparse(x)
    buf = io.BytesIO()
    torch.save(sparse, buf)
    buf.seek(0)
    again = torch.load(buf, weights_only=False)
    t = again[0].weight.wrapped_tensor
    assert set(vars(t)) == {"val", "idx", "nm_strides"}
    assert t.idx.dtype == torch.int16 and t.idx.shape[-1] == 1 and t.val.shape[-1] == 2
    assert torch.equal(again(x), y)
    w = sparse[0].weight
    w_cpu = w.to("cpu")
    assert isinstance(w_cpu.wrapped_tensor, sten.GroupedNMTensor) and w_cpu.wrapped_tensor.val.device.type == "cpu"
    w_back = w_cpu.to(cuda())
    assert torch.equal(w_back.wrapped_tensor.idx, w.wrapped_tensor.idx)
    half = w.to(torch.float16)
    assert half.wrapped_tensor.val.dtype == torch.float16 and torch.equal(half.wrapped_tensor.idx, w.wrapped_tensor.idx)
    assert w.shape == (48, 120) and w.dtype == torch.float32


def test_fp16_encoder_layer_shapes_run_through_the_kernels():
    """One BERT-large-shaped block of linears at 2:4 in fp16 (the configuration of the encoder benchmark)."""
    import sten_b200 as sten
    sten.set_dispatch_failure("raise")
    torch.manual_seed(0)
    block = torch.nn.Sequential(torch.nn.Linear(1024, 4096), torch.nn.GELU(), torch.nn.Linear(4096, 1024)).to(cuda()).half()
    sparse = _sparsify(block, 2, 4, 16)
    x = seeded_normal((4, 96, 1024), 9).to(cuda()).half()
    with torch.no_grad():
        y = sparse(x)
        dense = _densified_copy(sparse, block)
        yd = dense.float()(x.float())
    assert rel_fro(np_of(y), np_of(yd)) <= 1e-2


def test_row_shards_equal_slices_of_the_full_sparsified_weight():
    """Sparsifying a row slice gives exactly the tiles of that slice in the full result (tiles never interact), which is
    what makes row-sharding across GPUs exact; and the sharded layer on one rank is the plain kernel."""
    import sten_b200 as sten
    from sten_b200 import ops
    from sten_b200.sharded import ShardedGroupedNMLinear, row_shard_bounds
    M, K, n, m, g, R = 256, 1000, 2, 8, 16, 4
    w = seeded_normal((M, K), 21).to(cuda())
    full_val, full_idx = ops.sparsify(w.unsqueeze(0), n, m, g)
    C, cc, nb, nc = ops.geometry(M, K, n, m, g)
    fv = full_val.view(nc, nb, C, g, n)
    fi = full_idx.view(nc, nb, C, g, 1)
    bounds = row_shard_bounds(M, R, m)
    assert bounds == [0, 64, 128, 192, 256]
    for r in range(R):
        val, idx = ops.sparsify(w[bounds[r]:bounds[r + 1]].unsqueeze(0), n, m, g)
        lo, hi = bounds[r] // m, bounds[r + 1] // m
        assert torch.equal(val.view(nc, hi - lo, C, g, n), fv[:, lo:hi])
        assert torch.equal(idx.view(nc, hi - lo, C, g, 1), fi[:, lo:hi])
    x = seeded_normal((70, K), 22).to(cuda())
    shard = sten.GroupedNMTensor.from_dense(w, n, m, sparse_dim=0, group_size=g, group_dim=1)
    layer = ShardedGroupedNMLinear(shard, None, M)
    assert torch.equal(layer(x), ops.spmm(full_val, full_idx, M, K, n, m, g, x))


def test_weight_gradient_in_the_weight_layout_and_clone_layout():
    """set_weight_grad(..., WeightLayoutSparsifier, GroupedNMTensor): dW comes back packed in the weight's own layout (same
    idx object), equal to the dense dY^T X at the kept positions; clone_layout is the gather behind it."""
    import sten_b200 as sten
    sten.set_dispatch_failure("raise")
    dev = cuda()
    M, K, tokens, n, m, g = 96, 200, 64, 2, 4, 4
    torch.manual_seed(5)
    lin = torch.nn.Linear(K, M).to(dev)
    sb = sten.SparsityBuilder()
    sb.set_weight("weight", initial_sparsifier=sten.GroupedNMSparsifier(n, m, g), out_format=sten.GroupedNMTensor)
    sb.set_weight_grad("weight", inline_sparsifier=sten.WeightLayoutSparsifier(), tmp_format=sten.GroupedNMTensor,
                       external_sparsifier=sten.KeepAll(), out_format=sten.GroupedNMTensor)
    sparse = sb.get_sparse_model(lin)
    x = torch.randn(tokens, K, device=dev, requires_grad=True)
    dy = torch.randn(tokens, M, device=dev)
    sparse(x).backward(dy)
    gw = sparse.weight.grad
    assert isinstance(gw, sten.SparseTensorWrapper) and isinstance(gw.wrapped_tensor, sten.GroupedNMTensor)
    w_gnm, g_gnm = sparse.weight.wrapped_tensor, gw.wrapped_tensor
    assert g_gnm.idx is w_gnm.idx and g_gnm.val.shape == w_gnm.val.shape
    dense_dw = dy.t() @ x.detach()
    kept = w_gnm.clone_layout(torch.ones(M, K, device=dev)).to_dense() != 0      # the layout's positions
    want = torch.where(kept, dense_dw, torch.zeros_like(dense_dw))
    assert torch.allclose(g_gnm.to_dense(), want, rtol=1e-5, atol=1e-5)
    # exactly n of every m rows per column are kept, and dX is unaffected by the gradient format
    assert int(kept.sum()) == M * K * n // m
    dx_ref = dy @ w_gnm.to_dense()
    assert torch.allclose(x.grad, dx_ref, rtol=1e-4, atol=1e-4)
    # clone_layout on a 3-D layout (n:m along dim 2, groups along dim 1)
    t3 = sten.GroupedNMTensor.from_dense(torch.rand(3, 5, 17, device=dev), 2, 4, sparse_dim=2, group_size=2, group_dim=1)
    other = torch.rand(3, 5, 17, device=dev)
    cl = t3.clone_layout(other)
    mask3 = t3.to_dense() != 0
    assert torch.equal(cl.to_dense(), torch.where(mask3, other, torch.zeros_like(other)))


def test_fused_epilogues_in_a_small_bert_encoder():
    """fuse_linear_epilogues: dense+GELU and dense+residual+LayerNorm modules of a 2-layer BERT-shaped encoder with grouped
    n:m weights run through nmg_spmm_fused; the output equals the unfused sparse model's up to fp16 rounding, and the
    densified model's within the 16-bit tolerance."""
    import copy
    transformers = pytest.importorskip("transformers")
    import sten_b200 as sten
    sten.set_dispatch_failure("raise")
    dev = cuda()
    cfg = transformers.BertConfig(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, intermediate_size=512,
                                  vocab_size=1000, max_position_embeddings=128)
    torch.manual_seed(0)
    model = transformers.BertModel(cfg, add_pooling_layer=False).half().to(dev).eval()
    names = [n + ".weight" for n, mod in model.named_modules() if isinstance(mod, torch.nn.Linear) and "encoder.layer" in n]
    sb = sten.SparsityBuilder()
    for w in names:
        sb.set_weight(name=w, initial_sparsifier=sten.GroupedNMSparsifier(n=2, m=4, g=16), out_format=sten.GroupedNMTensor)
    sparse = sb.sparsify_model_inplace(copy.deepcopy(model))
    densified = copy.deepcopy(model)
    sp = dict(sparse.named_parameters())
    with torch.no_grad():
        for name, prm in densified.named_parameters():
            if name in names:
                prm.copy_(sp[name].wrapped_tensor.to_dense())
    ids = torch.randint(0, 1000, (12, 128), generator=torch.Generator().manual_seed(1)).to(dev)  # 1536 tokens: two-pass path

    def fwd(m):
        with torch.no_grad():
            return m.encoder(m.embeddings(input_ids=ids), attention_mask=None).last_hidden_state

    plain = fwd(sparse)
    assert sten.fuse_linear_epilogues(sparse) == 3 * cfg.num_hidden_layers  # attention output, intermediate, output per layer
    assert sten.fuse_linear_epilogues(sparse) == 0                          # idempotent
    fused = fwd(sparse)
    ref = fwd(densified)
    rel = lambda a, b: float((a.double() - b.double()).norm() / b.double().norm())
    assert rel(fused, plain) <= 5e-3 and rel(fused, ref) <= 1e-2 and rel(plain, ref) <= 1e-2
    # with gradients enabled the modules fall back to their own forward (the fused call has no autograd)
    x = model.embeddings(input_ids=ids).detach().requires_grad_(True)
    y = sparse.encoder(x, attention_mask=None).last_hidden_state
    y.float().sum().backward()
    assert x.grad is not None and bool(torch.isfinite(x.grad.float()).all())


def test_kept_expanded_weight_is_an_opt_in_with_the_same_numbers():
    """set_spmm_opt(kernel="sm100-expanded"): F.linear of a large batch multiplies the kept expanded weight (no expansion
    pass); same bits as the default two-pass call, which expands into its workspace first.  Small batches and fp32 weights
    are unaffected."""
    import sten_b200 as sten
    from sten_b200 import ops
    sten.set_dispatch_failure("raise")
    dev = cuda()
    M, K, tokens, n, m, g = 384, 520, 1536, 2, 4, 16
    torch.manual_seed(3)
    lin = torch.nn.Linear(K, M, device=dev, dtype=torch.float16)
    sb = sten.SparsityBuilder()
    sb.set_weight("weight", initial_sparsifier=sten.GroupedNMSparsifier(n, m, g), out_format=sten.GroupedNMTensor)
    sparse = sb.get_sparse_model(lin)
    gnm = sparse.weight.wrapped_tensor
    x = torch.randn(tokens, K, device=dev, dtype=torch.float16)
    with torch.no_grad():
        default = sparse(x)
        assert gnm.__dict__.get("_expanded_cache") is None
        gnm.set_spmm_opt(kernel="sm100-expanded")
        kept = sparse(x)
        assert gnm.__dict__.get("_expanded_cache") is not None
        assert torch.equal(kept, default)
        small = sparse(x[:100])
    ref = x.double() @ gnm.to_dense().double().t() + sparse.bias.double()
    assert float((kept.double() - ref).norm() / ref.norm()) <= 1e-2
    assert float((small.double() - ref[:100]).norm() / ref[:100].norm()) <= 1e-2
    res = torch.randn(tokens, M, device=dev, dtype=torch.float16)
    fused = sten.sparse_linear_fused(x, gnm, sparse.bias, activation="gelu", residual=res)
    want = torch.nn.functional.gelu(ref) + res.double()
    assert float((fused.double() - want).norm() / want.norm()) <= 1e-2
    assert set(gnm.__getstate__()) == {"val", "idx", "nm_strides"} and ops.read_status() == 0
