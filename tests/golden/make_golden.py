"""Regenerate the golden fixtures in this directory by running the REFERENCE's own code on the CPU.

Run where a checkout of SAI-Lab-NYU/LSVD is available:

    python tests/golden/make_golden.py /path/to/LSVD

It imports the reference's PyTorch quantisers and modules, and executes its Triton
kernels with Triton's CPU interpreter, on small seeded inputs; inputs and outputs
are stored as ``.npz`` files next to this script.  The fixtures travel with the
repository; the reference checkout does not.

Stand-ins needed to import the reference without its optional dependencies:
  * empty permissive packages for ``llava``, ``accelerate``, ``vlmeval``,
    ``qwen_vl_utils`` (imported at module scope by the reference, unused here);
  * ``fast_hadamard_transform.hadamard_transform(x, scale)``: the external CUDA
    extension is replaced by a Sylvester butterfly that computes in fp32 and returns
    the input dtype, which is that extension's documented behaviour;
  * Triton's autotuner is bypassed with one fixed configuration (it needs a GPU
    driver), and the three ``libdevice.fast_*`` intrinsics of the attention kernel,
    which the interpreter lacks, are replaced by exp2/log2, cos and sin.
"""
import os
import sys
import types
import importlib.abc
import importlib.machinery

os.environ["TRITON_INTERPRET"] = "1"
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("LSVD_REFERENCE", "")
if not os.path.isdir(REF):
    sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of SAI-Lab-NYU/LSVD>  (or set LSVD_REFERENCE)")
HERE = os.path.dirname(os.path.abspath(__file__))

import numpy as np
import torch
import transformers  # noqa: F401  (must be imported before the stub finder is installed)


class _Permissive(types.ModuleType):
    __path__ = []

    def __getattr__(self, k):
        if k.startswith("__"):
            raise AttributeError(k)
        if k.isupper():
            return -200
        if k[0].islower():
            import importlib
            try:
                return importlib.import_module(self.__name__ + "." + k)
            except Exception:
                pass
        return type(k, (), {})


class _Finder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    ROOTS = ("llava", "accelerate", "vlmeval", "qwen_vl_utils")

    def find_spec(self, name, path, target=None):
        if name.split(".")[0] in self.ROOTS:
            return importlib.machinery.ModuleSpec(name, self, is_package=True)

    def create_module(self, spec):
        return _Permissive(spec.name)

    def exec_module(self, m):
        pass


sys.meta_path.insert(0, _Finder())

fht = types.ModuleType("fast_hadamard_transform")


def _hadamard_transform(x, scale=1.0):
    n = x.shape[-1]
    assert n & (n - 1) == 0
    y = x.reshape(-1, n).float().clone()
    h = 1
    while h < n:
        y = y.view(-1, n // (2 * h), 2, h)
        y = torch.stack((y[:, :, 0] + y[:, :, 1], y[:, :, 0] - y[:, :, 1]), dim=2).reshape(-1, n)
        h *= 2
    return (y * float(scale)).reshape(x.shape).to(x.dtype)


fht.hadamard_transform = _hadamard_transform
sys.modules["fast_hadamard_transform"] = fht


import triton
import triton.language as tl


@triton.jit
def _powf(x, y):
    return tl.exp2(y * tl.log2(x + tl.zeros_like(y)))


@triton.jit
def _cosf(x):
    return tl.cos(x)


@triton.jit
def _sinf(x):
    return tl.sin(x)


def save(name, **arrs):
    out = {}
    for k, v in arrs.items():
        if isinstance(v, torch.Tensor):
            v = v.detach().cpu().numpy()
        out[k] = np.asarray(v)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print("wrote", name, {k: (v.shape, str(v.dtype)) for k, v in out.items()})


def edge_latents(T, H, R, g):
    """fp16 latents with the awkward rows in front: zeros, tiny, huge, exact .5 quotients."""
    x = torch.randn(T, H, R, generator=g).half()
    x[0] = 0
    x[1] = 1e-6
    x[2] = x[2] * 3000
    x[3, :, 0] = 128.0
    x[3, :, 1:] = torch.arange(R - 1).half()[None, :] + 0.5
    x[4] = -x[3]
    x[5] = x[5] * 1e-3
    x[6, :, 0] = 65504.0
    return x


# ------------------------------------------------------------------ kernels/ side
class Fixed:
    """Stands in for a triton.autotune object: launches the wrapped kernel with one fixed configuration."""

    def __init__(self, auto, **cfg):
        self.fn = auto.fn
        self.cfg = cfg
        self.best_config = types.SimpleNamespace(kwargs=cfg)

    def __getitem__(self, grid):
        gr = grid(self.cfg) if callable(grid) else grid
        return lambda *a, **k: self.fn[gr](*a, **k, **self.cfg)


def _kernels_side_imports():
    for d in ("layer_bench", os.path.join("layer_bench", "fd_kernel")):
        path = os.path.join(REF, "kernels", d)
        if path not in sys.path:
            sys.path.insert(0, path)
    tl.extra.cuda.libdevice.fast_powf = _powf
    tl.extra.cuda.libdevice.fast_cosf = _cosf
    tl.extra.cuda.libdevice.fast_sinf = _sinf


def gen_kernels_side():
    _kernels_side_imports()
    import benchmark_triton_int8_layer as bench
    from ffn_kernel import baseline_kernel
    import destindex_copy_quantize_latent as dcq
    import flash_int8_latent_per_head_decoding_rope_stage1 as s1
    import flash_latent_per_head_decoding_stage2 as s2

    g = torch.Generator().manual_seed(0)

    # 1. latent cache quantiser: PyTorch twin (normative) and the Triton append kernel
    T, H, R = 40, 3, 24
    x = edge_latents(T, H, R, g)
    q_t, s_t, _ = bench.quantize_latent_tensor(x, return_dequantized=False)
    dest = torch.randperm(64, generator=g)[:T].to(torch.int32)
    cache = torch.zeros(64, H, R, dtype=torch.int8)
    cache_s = torch.zeros(64, H, dtype=torch.float16)
    dcq.destindex_copy_quantize_latent(x, dest, cache, cache_s)
    save("latent_quant", x=x, q_torch=q_t, s_torch=s_t, dest_loc=dest, cache_triton=cache, scale_triton=cache_s)

    # 2. K up-factor quantiser
    wuk = (torch.randn(16, 96, generator=g) * 0.1).half()
    wuk[:, 0] = 0
    wq, ws = baseline_kernel.Int8AttentionBlock._quantize_wuk(None, wuk)
    save("wuk_quant", wuk=wuk, wuk_q=wq, wuk_scale=ws)

    # 3. decode attention: stage 1 + stage 2 in the interpreter, two fixed block configurations
    auto = s1._fwd_kernel_flash_int8_latent_decode_rope_stage1
    B, Hq, Hkv, D, Rk, Rv, S = 3, 4, 2, 32, 16, 32, 300
    q = torch.randn(B, Hq, D, generator=g).half()
    lk = torch.randn(B * S, Hkv, Rk, generator=g).half()
    lv = torch.randn(B * S, Hkv, Rv, generator=g).half()
    kq, ks, _ = bench.quantize_latent_tensor(lk, return_dequantized=False)
    vq, vs, _ = bench.quantize_latent_tensor(lv, return_dequantized=False)
    wukf = (torch.randn(Rk, Hkv * D, generator=g) * 0.1).half()
    wq, ws = baseline_kernel.Int8AttentionBlock._quantize_wuk(None, wukf)
    slots = torch.randperm(B * S, generator=g).to(torch.int32).view(B, S)       # non-identity slot map
    b_req = torch.tensor([2, 0, 1], dtype=torch.int32)
    b_len = torch.tensor([S, S - 37, 1], dtype=torch.int32)
    outs = {}
    for tag, cfg in (("a", dict(BLOCK_N=16, BLOCK_SEQ=256)), ("b", dict(BLOCK_N=32, BLOCK_SEQ=512))):
        s1._fwd_kernel_flash_int8_latent_decode_rope_stage1 = Fixed(auto, **cfg)
        BS = 256
        nblk = (S + BS - 1) // BS
        mid = torch.zeros(B, Hq, nblk, Rv, dtype=torch.float32)
        lse = torch.zeros(B, Hq, nblk, dtype=torch.float32)
        used = s1.flash_int8_latent_per_head_decode_rope_stage1(q, kq, ks, vq, vs, wq, ws, slots, b_req, b_len, S, mid, lse, BS)
        o = torch.zeros(B, Hq, Rv, dtype=torch.float16)
        s2.flash_decode_stage2(mid, lse, b_len, o, used)
        outs["o_" + tag] = o
    save("attn_rope_recon", q=q, cache_k=kq, scale_k=ks, cache_v=vq, scale_v=vs, wk_q=wq, wk_scale=ws,
         req_to_token=slots, b_req_idx=b_req, b_seq_len=b_len, **outs)


def gen_attention_block():
    """One decode step of the reference's whole Int8AttentionBlock (kernels/layer_bench/ffn_kernel/baseline_kernel.py:
    56-145) on the CPU: fp16 projections by PyTorch, append and attention kernels in the Triton interpreter.  The
    wrapper's scratch buffers, which it places on "cuda", are given to it on the CPU instead."""
    _kernels_side_imports()
    import functools
    import benchmark_triton_int8_layer as bench
    from ffn_kernel import baseline_kernel
    import flash_int8_latent_per_head_decoding_rope_stage1 as s1

    torch.manual_seed(11)
    g = torch.Generator().manual_seed(11)
    hidden, H, D, ratio = 128, 4, 32, 0.5
    blk = baseline_kernel.Int8AttentionBlock(hidden, H, D, ratio, device="cpu")
    blk.input_layernorm_weight.data = (1 + 0.1 * torch.randn(hidden, generator=g)).half()
    R = blk.rank_head
    lens = [40, 17, 1]
    B, S = len(lens), max(lens)
    N = B * S + 5

    class State:
        pass
    st = State()
    st.batch_size, st.max_len_in_batch = B, S
    st.b_seq_len = torch.tensor(lens, dtype=torch.int32)
    st.b_req_idx = torch.tensor([1, 2, 0], dtype=torch.int32)
    st.req_manager = State()
    st.req_manager.req_to_token_indexs = torch.randperm(N, generator=g)[:B * S].to(torch.int32).view(B, S)
    st.mem_index = st.req_manager.req_to_token_indexs[st.b_req_idx.long(), st.b_seq_len.long() - 1].contiguous()

    kq, ks, _ = bench.quantize_latent_tensor(torch.randn(N, H, R, generator=g).half(), return_dequantized=False)
    vq, vs, _ = bench.quantize_latent_tensor(torch.randn(N, H, R, generator=g).half(), return_dequantized=False)
    before = dict(cache_k=kq.clone(), scale_k=ks.clone(), cache_v=vq.clone(), scale_v=vs.clone())
    x = torch.randn(B, 1, hidden, generator=g).half()

    s1._fwd_kernel_flash_int8_latent_decode_rope_stage1 = Fixed(s1._fwd_kernel_flash_int8_latent_decode_rope_stage1,
                                                                BLOCK_N=16, BLOCK_SEQ=256)
    on_cpu = lambda shape, dtype, device=None: torch.zeros(*shape, dtype=dtype)
    baseline_kernel.token_decode_attention_flash_int8_latent_per_head_decoding_rope = functools.partial(
        baseline_kernel.token_decode_attention_flash_int8_latent_per_head_decoding_rope, alloc_tensor_func=on_cpu)
    y = blk(x, kq, ks, vq, vs, st)
    save("attention_block", x=x, y=y, num_heads=np.int64(H), head_dim=np.int64(D), rank_head=np.int64(R),
         down_proj_q=blk.down_proj_q.weight, down_proj_kv=blk.down_proj_kv.weight, o_proj=blk.o_proj.weight,
         up_proj_q=blk.up_proj_q, up_proj_k=blk.up_proj_k, up_proj_v=blk.up_proj_v,
         input_layernorm_weight=blk.input_layernorm_weight, wuk_q=blk.wuk_q, wuk_scale=blk.wuk_scale, wuvout=blk.wuvout,
         req_to_token=st.req_manager.req_to_token_indexs, b_req_idx=st.b_req_idx, b_seq_len=st.b_seq_len,
         mem_index=st.mem_index, cache_k_after=kq, scale_k_after=ks, cache_v_after=vq, scale_v_after=vs, **before)


def gen_mixffn():
    """The reference's mixffn W8A8 FFN (kernels/layer_bench/ffn_kernel/mix_ffn_kernel.py): a SwiGLUFFN from its seeded
    generator converted by ``MixedFFNGateUpDenseLatentFused.from_float`` and run through ``forward_stages`` with all
    eleven Triton kernels in the interpreter.  Each autotuned kernel runs the configuration with the smallest row-max
    tile, the one the wrappers size their scratch rows for."""
    _kernels_side_imports()
    from triton.runtime.autotuner import Autotuner

    def run_fixed(self, *args, **kwargs):
        cfg = min(self.configs, key=lambda c: (c.kwargs.get("BLOCK_R", 0) if "BLOCK_N" not in c.kwargs else 0,
                                               c.kwargs.get("BLOCK_N", 0), c.kwargs.get("BLOCK_M", 0)))
        self.best_config = cfg
        return self.fn.run(*args, **kwargs, **cfg.kwargs)
    Autotuner.run = run_fixed
    from ffn_kernel import mix_ffn_kernel as mk

    hidden, d_ffn, M = 512, 1024, 5
    torch.manual_seed(23)                      # the low-rank factors come from the global generator (:545-554)
    x, module = mk.make_ffn_inputs(1, M, hidden, d_ffn, seed=7, device="cpu", svd_ratio=0.5, rank_ratio=0.5, round_to=64)
    x[0, 3] = 0                                # a token of zeros: every scale falls to its floor
    mixed = mk.MixedFFNGateUpDenseLatentFused.from_float(module, 0.5, 0.5, 64)
    st = mixed.forward_stages(x)
    wts = {"norm_weight": mixed.norm_weight}
    for name in ("up", "gate", "down"):
        proj = getattr(mixed, name + "_proj")
        wts.update({name + "_a_q": proj.svd_branch.a_q, name + "_a_scale": proj.svd_branch.a_scale,
                    name + "_b_q": proj.svd_branch.b_q, name + "_b_scale": proj.svd_branch.b_scale,
                    name + "_q": proj.dense_branch.q, name + "_scale": proj.dense_branch.scale})
    stages = {"st_" + k: v for k, v in st.items() if isinstance(v, torch.Tensor)}
    save("mixffn", x=x, eps=np.float64(mixed.eps), fp16_up_w=module.up_proj.weight, fp16_gate_w=module.gate_proj.weight,
         fp16_down_w=module.down_proj.weight, **wts, **stages)


# ------------------------------------------------------------------ fake_quant/ side
def gen_fake_quant_side():
    for m in [k for k in sys.modules if k == "utils" or k.startswith("utils.")]:
        del sys.modules[m]
    sys.path.insert(0, os.path.join(REF, "fake_quant"))
    import torch.nn as nn
    from utils import quant_utils, hadamard_utils
    from utils.hybrid_ffn_utils import HybridSVDQuantFFN, _make_quant_linear
    from utils.svd_utils import SVDLinear

    g = torch.Generator().manual_seed(1)

    # 4. activation and weight quantisers
    xa = torch.randn(9, 64, generator=g).half()
    xa[0] = 0
    xa[1, :] = torch.linspace(-3, 3, 64).half()
    aq = quant_utils.ActQuantizer()
    aq.configure(bits=8, groupsize=-1, sym=True, clip_ratio=1.0)
    aq.find_params(xa)
    a_codes, a_scale = aq.quantize(xa)
    a_fake = aq(xa)
    W = (torch.randn(24, 64, generator=g) * 0.02).half()
    W[3] = 0
    wres = {}
    for tag, mse in (("rtn", False), ("mse", True)):
        wq = quant_utils.WeightQuantizer()
        wq.configure(8, perchannel=True, sym=True, mse=mse)
        wq.find_params(W)
        fake, codes, scale = wq.fake_quantize(W)
        wres["w_codes_" + tag], wres["w_scale_" + tag], wres["w_fake_" + tag] = codes, scale, fake
    save("fq_quantizers", x=xa, a_codes=a_codes, a_scale=a_scale[:, 0], a_fake=a_fake, W=W, **wres)

    # 5. Hadamard: power-of-two and the K = 172, 108 factored forms, plus the factors themselves (bit-packed)
    res = {}
    for n in (64, 172 * 4, 108 * 8):
        hk, K = hadamard_utils.get_hadK(n)
        xh = torch.randn(5, n, generator=g).half()
        res[f"x_{n}"] = xh
        res[f"y_{n}"] = hadamard_utils.matmul_hadU_cuda(xh, hk, K)
        res[f"K_{n}"] = K
    for K in (172, 108):
        hk, _ = hadamard_utils.get_hadK(K * 64)
        res[f"had{K}_bits"] = np.packbits((hk.numpy() > 0).astype(np.uint8))
    # input rotation: x @ random_hadamard_matrix(n) with the sign vector recovered from the matrix
    torch.manual_seed(7)
    Q = hadamard_utils.random_hadamard_matrix(128, "cpu")                      # float64
    sign = torch.sign(Q[:, 0]).float()                                        # column 0 of H is all ones
    xr = torch.randn(6, 128, generator=g).half()
    res["rot_x"], res["rot_sign"], res["rot_y"] = xr, sign, (xr.double() @ Q).half()
    save("hadamard", **res)

    # 6. the hybrid FFN module itself, fp16 on the CPU, with every sub-module output captured
    d_in, d_ffn, r = 128, 172 * 16, 64
    n_svd = d_ffn // 2
    n_q = d_ffn - n_svd

    def rtn_(lin):
        wq = quant_utils.WeightQuantizer()
        wq.configure(8, perchannel=True, sym=True, mse=False)
        wq.find_params(lin.weight.data)
        fake, codes, scale = wq.fake_quantize(lin.weight.data)
        lin.weight.data = wq.quantize(lin.weight.data).to(lin.weight.dtype)
        return codes.to(torch.int8), scale.flatten().float()

    def svd_lin():
        m = SVDLinear.__new__(SVDLinear)
        nn.Module.__init__(m)
        m.BLinear = nn.Linear(d_in, r, bias=False)
        m.ALinear = nn.Linear(r, n_svd, bias=False)
        m.is_ma_hack = False
        m.original_linear = None
        m.is_per_head_svd = False
        m.BLinear.weight.data = torch.randn(r, d_in, generator=g) * 0.1
        m.ALinear.weight.data = torch.randn(n_svd, r, generator=g) * 0.1
        m = m.half()
        m.BLinear = quant_utils.ActQuantWrapper(m.BLinear)
        return m

    ref_lin = nn.Linear(d_in, d_ffn, bias=False).half()
    g_svd, u_svd = svd_lin(), svd_lin()
    g_q = _make_quant_linear(torch.randn(n_q, d_in, generator=g) * 0.1, d_in, ref_lin)
    u_q = _make_quant_linear(torch.randn(n_q, d_in, generator=g) * 0.1, d_in, ref_lin)
    down = quant_utils.ActQuantWrapper(nn.Linear(d_ffn, d_in, bias=False).half())
    down.module.weight.data = (torch.randn(d_in, d_ffn, generator=g) * 0.05).half()
    had_K, K = hadamard_utils.get_hadK(d_ffn)
    ffn = HybridSVDQuantFFN(g_svd, u_svd, g_q, u_q, down, torch.arange(d_ffn), n_svd, had_K=had_K, K=K)
    wts = {}
    for name, lin in (("Ug", g_svd.BLinear.module), ("Uu", u_svd.BLinear.module), ("Vg", g_svd.ALinear),
                      ("Vu", u_svd.ALinear), ("Wg", g_q.module), ("Wu", u_q.module), ("Wd", down.module)):
        wts[name + "_q"], wts[name + "_s"] = rtn_(lin)
    for wmod in (g_svd.BLinear, u_svd.BLinear, g_q, u_q, down):
        wmod.quantizer.configure(bits=8, groupsize=-1, sym=True, clip_ratio=1.0)
    for wmod in (g_svd.BLinear, u_svd.BLinear):
        wmod.out_quantizer.configure(bits=8, groupsize=-1, sym=True, clip_ratio=1.0)
    cap = {}

    def hook(tag):
        def f(mod, inp, out):
            cap[tag + "_in"] = inp[0].detach().clone()
            cap[tag + "_out"] = out.detach().clone()
        return f

    g_svd.BLinear.register_forward_hook(hook("latg"))
    u_svd.BLinear.register_forward_hook(hook("latu"))
    g_svd.register_forward_hook(hook("gsvd"))
    u_svd.register_forward_hook(hook("usvd"))
    g_q.register_forward_hook(hook("grtn"))
    u_q.register_forward_hook(hook("urtn"))
    down.register_forward_hook(hook("down"))
    down.module.register_forward_hook(hook("downlin"))
    x = torch.randn(7, d_in, generator=g).half()
    with torch.no_grad():
        y = ffn(x)
    save("hybrid_ffn", x=x, y=y, K=K, had_bits=np.packbits((had_K.numpy() > 0).astype(np.uint8)),
         latg=cap["latg_out"], latu=cap["latu_out"], g_svd=cap["gsvd_out"], u_svd=cap["usvd_out"],
         g_rtn=cap["grtn_out"], u_rtn=cap["urtn_out"], h=cap["down_in"], h_fakeq=cap["downlin_in"], **wts)


def gen_partial_hadamard():
    """ActQuantWrapper with online_partial_had (the Hadamard across heads in front of o_proj,
    fake_quant/utils/quant_utils.py:302-317) followed by its A8 input quantiser: the tensor the wrapped Linear sees."""
    for m in [k for k in sys.modules if k == "utils" or k.startswith("utils.")]:
        del sys.modules[m]
    sys.path.insert(0, os.path.join(REF, "fake_quant"))
    import torch.nn as nn
    from utils import quant_utils
    g = torch.Generator().manual_seed(5)
    H, D = 32, 16
    x = torch.randn(6, H * D, generator=g).half()
    x[2] = 0
    lin = nn.Linear(H * D, 8, bias=False).half()
    wrap = quant_utils.ActQuantWrapper(lin)
    wrap.online_partial_had, wrap.had_dim, wrap.K = True, D, 1
    seen = {}
    lin.register_forward_pre_hook(lambda mod, inp: seen.__setitem__("x", inp[0].detach().clone()))
    wrap.quantizer.configure(bits=16)
    wrap(x)
    rotated = seen["x"]
    wrap.quantizer.configure(bits=8, groupsize=-1, sym=True, clip_ratio=1.0)
    wrap(x)
    # a head count that is not a power of two (28: Qwen2-VL-7B): the had_K @ x form of the same wrapper
    from utils import hadamard_utils
    H2 = 28
    hk, K2 = hadamard_utils.get_hadK(H2)
    assert K2 == H2
    x2 = torch.randn(5, H2 * D, generator=g).half()
    lin2 = nn.Linear(H2 * D, 8, bias=False).half()
    wrap2 = quant_utils.ActQuantWrapper(lin2)
    wrap2.online_partial_had, wrap2.had_dim, wrap2.K, wrap2.had_K = True, D, K2, hk
    seen2 = {}
    lin2.register_forward_pre_hook(lambda mod, inp: seen2.__setitem__("x", inp[0].detach().clone()))
    wrap2.quantizer.configure(bits=16)
    wrap2(x2)
    save("partial_hadamard", x=x, heads=np.int64(H), head_dim=np.int64(D), rotated=rotated, fake_quant=seen["x"],
         x28=x2, had28=hk.to(torch.int8), rotated28=seen2["x"])


def gen_modules():
    """SVDLinear (ragged and uniform per-head forms), ActQuantWrapper in its rotation / quantiser settings, and the two
    on-disk formats of the hybrid FFN: a channel-group JSON and a --save_qmodel_path style checkpoint."""
    for m in [k for k in sys.modules if k == "utils" or k.startswith("utils.")]:
        del sys.modules[m]
    sys.path.insert(0, os.path.join(REF, "fake_quant"))
    import json
    import torch.nn as nn
    from utils import quant_utils, hadamard_utils, svd_utils
    from utils.svd_utils import SVDLinear
    from utils import hybrid_ffn_utils as hf
    g = torch.Generator().manual_seed(11)

    # ---- SVDLinear, per head with a rank split (svd_utils.py:185-233, 1978-2015) and uniform (:234-268, 2017-2027)
    H, cout, cin = 4, 16, 64
    ranks = [16, 32, 16, 48]
    U = [torch.randn(cout, r, generator=g).half() for r in ranks]
    S = [torch.rand(r, generator=g).half() + 0.5 for r in ranks]
    V = [(torch.randn(cin, r, generator=g) * 0.2).half() for r in ranks]
    bias = (torch.randn(H * cout, generator=g) * 0.1).half()
    res = {}
    for fuse in ("UV", "U", "V"):
        m = SVDLinear(U, S, V, bias=bias if fuse == "UV" else None, sigma_fuse=fuse, is_per_head_svd=True, rank_split=ranks)
        x = torch.randn(2, 3, cin, generator=g).half()
        res[f"ragged_{fuse}_x"], res[f"ragged_{fuse}_y"] = x, m(x)
        res[f"ragged_{fuse}_B"] = m.BLinear.weight.data
        res[f"ragged_{fuse}_A"] = torch.cat([a.data.reshape(-1) for a in m.ALinear])
    r = 32
    Uu = torch.randn(H, cout, r, generator=g).half()
    Su = torch.rand(H, r, generator=g).half() + 0.5
    Vu = (torch.randn(H, cin, r, generator=g) * 0.2).half()
    m = SVDLinear(Uu, Su, Vu, sigma_fuse="UV", is_per_head_svd=True)
    xu = torch.randn(1, 5, cin, generator=g).half()
    res.update(uni_U=Uu, uni_S=Su, uni_V=Vu, uni_x=xu, uni_y=m(xu), uni_B=m.BLinear.weight.data, uni_A=m.ALinear.data)
    save("svd_linear", ranks=np.array(ranks), bias=bias, U=torch.cat([u.reshape(-1) for u in U]), S=torch.cat(S),
         V=torch.cat([v.reshape(-1) for v in V]), cout=np.int64(cout), cin=np.int64(cin), **res)

    # ---- ActQuantWrapper (quant_utils.py:225-340): Linear weights int8 fake-quantised by the reference's own RTN
    def rtn_(lin, mse=False):
        wq = quant_utils.WeightQuantizer()
        wq.configure(8, perchannel=True, sym=True, mse=mse)
        wq.find_params(lin.weight.data)
        lin.weight.data = wq.quantize(lin.weight.data).to(lin.weight.dtype)
        return wq

    res = {}

    def case(tag, n_in, n_out, tokens, with_bias=False, out_bits=16, setup=None, w16=False):
        lin = nn.Linear(n_in, n_out, bias=with_bias).half()
        lin.weight.data = (torch.randn(n_out, n_in, generator=g) * 0.05).half()
        if with_bias:
            lin.bias.data = (torch.randn(n_out, generator=g) * 0.1).half()
        if not w16:
            rtn_(lin)
        w = quant_utils.ActQuantWrapper(lin)
        if setup is not None:
            setup(w)
        w.quantizer.configure(bits=8, groupsize=-1, sym=True, clip_ratio=1.0)
        if out_bits < 16:
            w.out_quantizer.configure(bits=out_bits, groupsize=-1, sym=True, clip_ratio=1.0)
        x = torch.randn(2, tokens, n_in, generator=g).half()
        x[0, 0] = 0
        res[tag + "_x"], res[tag + "_W"], res[tag + "_y"] = x, lin.weight.data, w(x)
        if with_bias:
            res[tag + "_b"] = lin.bias.data
        return w

    case("plain", 96, 48, 3, with_bias=True, out_bits=8)
    case("w16", 96, 48, 3, w16=True)

    def full(w):
        w.online_full_had = True
        w.had_K, w.K = hadamard_utils.get_hadK(w.in_features)
        if w.K > 1:
            res["had%d" % w.K] = w.had_K.to(torch.int8)

    case("full64", 64, 32, 4, setup=full)
    case("full768", 768, 32, 4, setup=full)

    def full32(w):
        full(w)
        w.fp32_had = True

    case("full64_fp32", 64, 32, 4, setup=full32)

    def partial(w):
        w.online_partial_had, w.had_dim, w.K = True, 16, 1

    case("partial", 8 * 16, 32, 4, setup=partial)

    def rnd(w):
        torch.manual_seed(3)
        w.online_random_had = True
        w.had_K = hadamard_utils.random_hadamard_matrix(w.in_features, "cpu").half()
        res["random_Q"] = w.had_K

    case("random", 128, 32, 4, setup=rnd)
    wr = case("many", 96, 48, 80, with_bias=True)          # more than 64 tokens: the prefill-sized product
    save("act_quant_wrapper", **res)

    # ---- channel groups: the selector's result in the layout the analysis pass writes (hybrid_ffn_utils.py:2774-2801)
    d_in, d_ffn, rank = 64, 192, 32
    n_svd = d_ffn // 2
    Wg = torch.randn(d_ffn, d_in, generator=g) * 0.1
    Wu = torch.randn(d_ffn, d_in, generator=g) * 0.1
    # the selector compares closed-form error proxies (hybrid_ffn_utils.py:156-176): rows with one large entry have a
    # coarse quantisation step and go to the SVD group; with the 2-bit error model more than n_svd rows qualify and the
    # cap keeps the n_svd with the largest margin
    spike = torch.randint(0, d_in, (d_ffn,), generator=g)
    rows = torch.arange(0, d_ffn, 2)
    Wg[rows, spike[rows]] *= 6
    Wu[rows, spike[rows]] *= 6
    Wd = torch.randn(d_in, d_ffn, generator=g) * 0.1
    calib = torch.randn(32, d_in, generator=g)
    svd_idx, quant_idx, perm = hf.select_svd_channels(Wg, Wu, Wd, n_svd, calib_inps=calib, svd_rank=rank, w_bits=2, w_sym=True)
    assert 0 < len(svd_idx) < d_ffn and len(svd_idx) % 16 == 0, len(svd_idx)
    order = [int(v) for v in torch.randperm(d_ffn, generator=g)[:150]]
    groups = {"layers": {}}
    for idx in (0, 1):
        entry = {"svd_idx": svd_idx, "quant_idx": quant_idx, "perm": perm.tolist(), "n_svd": len(svd_idx), "svd_rank": rank,
                 "d_ffn": d_ffn, "d_in": d_in}
        if idx == 1:
            entry["greedy_accept_order"] = order
        groups["layers"][str(idx)] = entry
    path = os.path.join(HERE, "channel_groups.json")
    with open(path, "w") as f:
        json.dump(groups, f, indent=2)
    back = hf.load_channel_groups(path)                      # the reference reads its own layout back
    assert back["layers"]["0"]["perm"] == perm.tolist()
    print("wrote channel_groups.json", len(svd_idx), len(quant_idx))

    # ---- checkpoint: a layer whose mlp is the reference's HybridSVDQuantFFN, quantised by the loop of rtn_fwrd
    # (gptq_utils.py:1168-1200) with the MSE clip search on, saved the way --save_qmodel_path does
    # (main_llava_next_hybrid_ffn.py:365-375)
    n_q = d_ffn - len(svd_idx)

    def svd_lin(n_out):
        m = SVDLinear.__new__(SVDLinear)
        nn.Module.__init__(m)
        m.BLinear = nn.Linear(d_in, rank, bias=False)
        m.ALinear = nn.Linear(rank, n_out, bias=False)
        m.is_ma_hack, m.original_linear, m.is_per_head_svd = False, None, False
        m.BLinear.weight.data = torch.randn(rank, d_in, generator=g) * 0.1
        m.ALinear.weight.data = torch.randn(n_out, rank, generator=g) * 0.1
        m = m.half()
        m.BLinear = quant_utils.ActQuantWrapper(m.BLinear)
        return m

    ref_lin = nn.Linear(d_in, d_ffn, bias=False).half()
    g_svd, u_svd = svd_lin(len(svd_idx)), svd_lin(len(svd_idx))
    g_q = hf._make_quant_linear(torch.randn(n_q, d_in, generator=g) * 0.1, d_in, ref_lin)
    u_q = hf._make_quant_linear(torch.randn(n_q, d_in, generator=g) * 0.1, d_in, ref_lin)
    down = quant_utils.ActQuantWrapper(nn.Linear(d_ffn, d_in, bias=False).half())
    down.module.weight.data = (torch.randn(d_in, d_ffn, generator=g) * 0.05).half()
    had_K, K = hadamard_utils.get_hadK(d_ffn)
    mlp = hf.HybridSVDQuantFFN(g_svd, u_svd, g_q, u_q, down, perm, len(svd_idx), had_K=had_K, K=K)

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.mlp = mlp

    class Inner(nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = nn.ModuleList([Layer()])

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.model = Inner()

    model = Model()
    quantizers = {}
    for i, layer in enumerate(model.model.layers):
        for name in hf.hybrid_ffn_rtn_targets():
            module = svd_utils.rgetattr(layer, name)
            qz = quant_utils.WeightQuantizer()
            qz.configure(8, perchannel=True, sym=True, mse=True)
            W = module.weight.data
            qz.find_params(W)
            module.weight.data = qz.quantize(W).to(device=W.device, dtype=W.dtype)
            quantizers[f"model.layers.{i}.{name}"] = qz.cpu()
    torch.save({"w_quantizers": quantizers, "model": model.state_dict()}, os.path.join(HERE, "qmodel_ffn.pt"))
    for wmod in (g_svd.BLinear, u_svd.BLinear, g_q, u_q, down):
        wmod.quantizer.configure(bits=8, groupsize=-1, sym=True, clip_ratio=1.0)
    for wmod in (g_svd.BLinear, u_svd.BLinear):
        wmod.out_quantizer.configure(bits=8, groupsize=-1, sym=True, clip_ratio=1.0)
    x = torch.randn(5, d_in, generator=g).half()
    scales = {k: v.scale.flatten().float() for k, v in quantizers.items()}
    save("qmodel_ffn_io", x=x, y=mlp(x), **{k.replace(".", "__"): v for k, v in scales.items()})
    print("wrote qmodel_ffn.pt", os.path.getsize(os.path.join(HERE, "qmodel_ffn.pt")), "bytes")


if __name__ == "__main__":
    with torch.no_grad():
        only = {"partial_hadamard": gen_partial_hadamard, "attention_block": gen_attention_block, "mixffn": gen_mixffn,
                "modules": gen_modules}
        if len(sys.argv) > 2 and sys.argv[2] in only:
            only[sys.argv[2]]()
            sys.exit(0)
        gen_kernels_side()
        gen_attention_block()
        gen_mixffn()
        gen_fake_quant_side()
        gen_partial_hadamard()
