"""Load a kernel spec, bind it to the sm_100a library and check it against the reference.

Mirrors the seams of python/cleave/runtime/compile.py: ``_load_main_kernel_from_code`` execs the
module text exactly as the reference does, ``_compile`` returns a callable with the TileLang
JIT kernel's facade (``adapter``, ``get_kernel_source``), ``check_code`` is the picklable
top-level function a worker runs. Nothing is compiled at run time: the kernels were built
ahead of time into ``libcleave_b200.so``; a missing library is a hard error.
"""

from __future__ import annotations

import tempfile
from types import SimpleNamespace

from ..codegen import B200CodeGen, KernelSpec
from ..core.errors import CompileError
from .validate import DEFAULT_TOLERANCE, BenchOptions, Tolerance, _check_kernel, _stage


def _load_main_kernel_from_code(code_str):
    import importlib.util
    import uuid

    with tempfile.NamedTemporaryFile(suffix=".py", mode="w") as f:
        f.write(code_str)
        f.flush()
        module_name = f"tmp_module_{uuid.uuid4().hex}"
        spec = importlib.util.spec_from_file_location(module_name, f.name)
        tmp_module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(tmp_module)  # type: ignore
        main_kernel = tmp_module.main_kernel
        # specs are frozen dataclasses: the per-load annotations live beside them
        object.__setattr__(main_kernel, "_cache_source_hint", code_str)
        object.__setattr__(main_kernel, "_cleave_pass_configs", getattr(tmp_module, "PASS_CONFIGS", {}))
    return main_kernel


class _Buffer(SimpleNamespace):
    pass


class _Adapter:
    """What callers read off a compiled kernel: ``prim_func.params``, ``prim_func.buffer_map[param]
    .name/.shape/.dtype``, ``result_idx``, ``params``, ``dynamic_symbolic_map``."""

    def __init__(self, spec: KernelSpec, out_idx):
        tensors = [p for p in spec.params if p.role != "scalar"]
        handles = [SimpleNamespace(name=p.name) for p in tensors]
        self.params = [_Buffer(name=p.name, shape=tuple(p.dims), dtype=p.dtype) for p in tensors]
        self.prim_func = SimpleNamespace(params=handles, buffer_map=dict(zip(map(id, handles), self.params)))
        # buffer_map is keyed by the handle object, as TVM's is
        self.prim_func.buffer_map = _HandleMap(handles, self.params)
        n = len(tensors)
        self.result_idx = None if out_idx is None else [i % n for i in out_idx]
        dyn = {}
        for bi, p in enumerate(tensors):
            for di, d in enumerate(p.dims):
                if isinstance(d, str):
                    dyn.setdefault(d, (bi, di))
        self.dynamic_symbolic_map = dyn


class _HandleMap(dict):
    def __init__(self, handles, buffers):
        super().__init__()
        self._by_id = {id(h): b for h, b in zip(handles, buffers)}

    def get(self, handle, default=None):
        return self._by_id.get(id(handle), default)

    def __getitem__(self, handle):
        return self._by_id[id(handle)]


class B200Kernel:
    """``kernel(*inputs)`` with ``out_idx``: allocates and returns the trailing outputs (a tensor,
    or a list); with ``out_idx=None`` the outputs are caller-owned trailing arguments."""

    def __init__(self, spec: KernelSpec, out_idx):
        from .. import _lib

        _lib.lib()  # fail now, loudly, if the sm_100a library is not built
        self.spec, self.out_idx = spec, None if out_idx is None else list(out_idx)
        self.adapter = _Adapter(spec, out_idx)
        self._source = getattr(spec, "_cache_source_hint", None) or B200CodeGen().gen(spec)

    def get_kernel_source(self) -> str:
        return self._source

    def _alloc_outputs(self, tensors):
        import torch

        from .reference import torch_dtype

        names = [p for p in self.spec.params if p.role == "input"]
        bound = {}
        for p, t in zip(names, tensors):
            for d, n in zip(p.dims, t.shape):
                if isinstance(d, str):
                    bound.setdefault(d, int(n))
        device = tensors[0].device
        return [torch.empty([bound[d] if isinstance(d, str) else int(d) for d in p.dims],
                            dtype=torch_dtype(p.dtype), device=device) for p in self.spec.outputs]

    def _two_stage(self, ins, outs):
        """One stage of the two-stage form of a split (the reference's partial / combine kernels)."""
        from .. import ops

        s = self.spec
        if s.family == "split_combine":
            axes = s.attrs["axes"]
            if s.attrs.get("divide"):
                num, den = ins[s.attrs["num"]], ins[s.attrs["den"]]
                ops.split_combine(num, den, axis=axes[s.attrs["num"]], out=outs[0])
            else:
                ops.split_combine(ins[0], axis=axes[0], out=outs[0])
            return
        a = s.by_role(ins)
        if s.family == "matmul":
            ops.matmul_split_partial(a["x"], a["w"], s.split, out=outs[0])
        elif s.family == "attention_decode" and s.dims["SQ"] == 1:
            d, hq = s.dims["D"], s.dims["HQ"]
            # the two outputs in the plan's own order: the weighted values (D per row) and the weight sums
            o_out = next(o for o in outs if o.numel() == hq * s.split * d)
            l_out = next(o for o in outs if o.numel() == hq * s.split)
            ops.attention_split_partial(a["q"], a["k"], a["v"], s.split, s.attrs.get("scale"), shift=s.attrs.get("shift"),
                                        o_part=o_out.view(hq, s.split, d), l_part=l_out.view(hq, s.split))
        else:
            raise CompileError(f"{s.family}: the partial stage of a two-stage split has no kernel; pass the "
                               "[partial, combine] pair to the code generator for one fused launch")

    def __call__(self, *args):
        from .. import ops

        s = self.spec
        n_in = len(s.inputs)
        if self.out_idx is None:
            if len(args) != n_in + len(s.outputs):
                raise TypeError(f"{s.family}: expected {n_in} inputs and {len(s.outputs)} outputs, got {len(args)}")
            ins, outs = list(args[:n_in]), list(args[n_in:])
        else:
            if len(args) != n_in:
                raise TypeError(f"{s.family}: expected {n_in} inputs, got {len(args)}")
            ins = list(args)
            outs = self._alloc_outputs([a for a, p in zip(ins, s.inputs) if p.role == "input"])
        split, mc = (s.split if s.split > 1 else 0), int(s.attrs.get("max_ctas", 0))
        f = s.family
        if s.role != "main":
            self._two_stage(ins, outs)
            return None if self.out_idx is None else (outs[0] if len(outs) == 1 else outs)
        a = s.by_role(ins)   # the library's name for every input, whatever the parameters are called
        if f == "matmul":
            ops.matmul(a["x"], a["w"], split_k=split, out=outs[0].view(a["x"].shape[0], -1), max_ctas=mc)
        elif f == "rmsnorm_matmul":
            ops.rmsnorm_matmul(a["x"], a["w"], eps=float(s.attrs.get("eps", 0.0)), gamma=a.get("gamma"), split_k=split,
                               out=outs[0].view(a["x"].shape[0], -1), max_ctas=mc)
        elif f == "swiglu":
            ops.swiglu(a["x"], a["w0"], a["w1"], split_k=split, out=outs[0].view(a["x"].shape[0], -1), max_ctas=mc)
        elif f == "attention_decode":
            # the same static attention family: few query rows stream KV through the split-KV decode kernel,
            # a query tile's worth of rows (the "prefill" shapes) runs QK^T and PV on tcgen05
            if s.dims["SQ"] >= 64 and s.dims["D"] in (64, 128) and split <= 1:
                ops.attention_prefill(a["q"], a["k"], a["v"], s.attrs.get("scale"), out=outs[0])
            else:
                ops.attention_decode(a["q"], a["k"], a["v"], s.attrs.get("scale"), out=outs[0], max_ctas=mc)
        elif f == "matmul_matmul":
            ops.matmul_matmul(a["q"], a["k"], a["v"], out=outs[0])
        elif f == "qknorm_attention":
            ops.qknorm_attention(a["q"], a["k"], a["v"], s.attrs.get("scale"), eps=float(s.attrs.get("eps", 0.0)),
                                 out=outs[0])
        elif f == "matmul_rowsum":
            ops.matmul_rowsum(a["x"], a["w"], out=outs[0])
        elif f == "lora":
            ops.lora(a["x"], a["w"], a["a"], a["b"], out=outs[0])
        elif f == "mla_decode":
            ops.mla_decode(a["q"], a["kv"], a["q_pe"], a["k_pe"], float(s.attrs["scale"]), out=outs[0], max_ctas=mc)
        elif f == "gqa_paged_decode":
            last = ins[5] if s.dims["page_size"] != 1 else None
            ops.gqa_paged_decode(ins[0], ins[1], ins[2], ins[3], ins[4], last, float(ins[-1]), out=outs[0],
                                 lse=outs[1], max_ctas=mc)
        elif f == "mla_paged_decode":
            ops.mla_paged_decode(ins[0], ins[1], ins[2], ins[3], ins[4], ins[5], float(ins[6]), out=outs[0],
                                 lse=outs[1], max_ctas=mc)
        elif f == "mla_paged_prefill":
            ops.mla_paged_prefill(ins[0], ins[1], ins[2], ins[3], ins[4], ins[5], ins[6], float(ins[7]), out=outs[0],
                                  lse=outs[1])
        elif f == "gqa_ragged_prefill":
            ops.gqa_ragged_prefill(ins[0], ins[1], ins[2], ins[3], ins[4], float(ins[5]), out=outs[0], lse=outs[1])
        elif f == "gqa_paged_prefill":
            ops.gqa_paged_prefill(ins[0], ins[1], ins[2], ins[3], ins[4], ins[5], float(ins[6]), out=outs[0], lse=outs[1])
        else:  # pragma: no cover - from_dict rejects unknown families
            raise CompileError(f"unknown kernel family {f!r}")
        if self.out_idx is None:
            return None
        return outs[0] if len(outs) == 1 else outs


def _compile(main_kernel, out_idx):
    """Bind a loaded spec to the library (the reference's ``tl.compile`` seam)."""
    if not isinstance(main_kernel, KernelSpec):
        raise CompileError(f"main_kernel must be a KernelSpec, got {type(main_kernel).__name__}")
    return B200Kernel(main_kernel, out_idx)


def graph_out_indices(spec: KernelSpec) -> list:
    """Negative indices of the outputs among the tensor parameters (trailing)."""
    n = len(spec.outputs)
    return list(range(-n, 0))


def build_candidate_code(cand) -> str:
    """Kernel-spec text for one candidate (a KernelSpec, a scheduled plan, or a TileDict-like
    object with ``flat_graph``): the default ``build_fn``."""
    return B200CodeGen().gen(getattr(cand, "spec", cand))


def build_inputs_and_reference(spec: KernelSpec, device="cuda", seed=None):
    """``(inputs_by_name, [reference tensors], out_idx)`` for a static family: seeded N(0,1)
    inputs (weights scaled by 1/sqrt(K), gamma = 1 + 0.1 N(0,1)) and the torch fp32 reference cast to
    the storage dtype."""
    import torch

    from . import reference as R

    dt = R.torch_dtype(spec.dtype)
    g = torch.Generator(device="cpu").manual_seed(R.fingerprint_seed(spec) if seed is None else seed)
    d = spec.dims
    f_ = spec.family
    if spec.role != "main":
        return _two_stage_inputs_and_reference(spec, dt, g, device)
    inputs, by_role = {}, {}
    for p, base in zip(spec.inputs, spec.input_roles()):
        shape = [int(x) for x in p.dims]
        if base == "gamma":
            t = 1 + 0.1 * torch.randn(shape, generator=g)
        elif base in ("w", "w0", "w1") or (f_ == "lora" and base == "a"):
            # weights scaled so that products stay O(1): intermediates (LoRA's X @ A) are 16-bit on the GPU
            t = torch.randn(shape, generator=g) / d["K"] ** 0.5
        elif f_ == "lora" and base == "b":
            t = torch.randn(shape, generator=g) / d["R"] ** 0.5
        elif f_ == "matmul_matmul" and base == "v":
            # 16-bit scores feed the second product: keep the output O(1) so that their rounding stays
            # inside the absolute tolerance (with N(0,1) values the output has magnitude sqrt(SKV * D))
            t = torch.randn(shape, generator=g) / (d["SKV"] * d["D"]) ** 0.5
        else:
            t = torch.randn(shape, generator=g)
        inputs[p.name] = by_role[base] = t.to(dt).to(device)
    v = by_role.__getitem__
    f = spec.family
    if f == "matmul":
        ref = R.matmul(v("x"), v("w"))
    elif f == "rmsnorm_matmul":
        ref = R.rmsnorm_matmul(v("x"), v("w"), float(spec.attrs.get("eps", 0.0)), by_role.get("gamma"))
    elif f == "swiglu":
        ref = R.swiglu(v("x"), v("w0"), v("w1"))
    elif f == "attention_decode":
        ref = R.attention(v("q"), v("k"), v("v"), spec.attrs.get("scale"))
    elif f == "mla_decode":
        ref = R.mla_decode(v("q"), v("kv"), v("q_pe"), v("k_pe"), float(spec.attrs["scale"]))
    elif f == "matmul_matmul":
        ref = R.matmul_matmul(v("q"), v("k"), v("v"))
    elif f == "qknorm_attention":
        ref = R.qknorm_attention(v("q"), v("k"), v("v"), float(spec.attrs.get("eps", 0.0)), spec.attrs.get("scale"))
    elif f == "matmul_rowsum":
        ref = R.matmul_rowsum(v("x"), v("w"))
    elif f == "lora":
        ref = R.lora(v("x"), v("w"), v("a"), v("b"))
    else:
        raise CompileError(f"{f}: dynamic operators are validated over workloads, not one static reference")
    return inputs, [ref.to(dt)], graph_out_indices(spec)


def _two_stage_inputs_and_reference(spec: KernelSpec, dt, g, device):
    """Inputs and torch fp32 references of a partial or combine stage. A partial stage is checked against the
    per-split results themselves (as the reference checks its partial kernels, against the partial graph's own
    outputs), a combine stage on random partials."""
    import torch

    from . import reference as R

    inputs, by_role = {}, {}
    d = spec.dims
    if spec.family == "split_combine":
        for i, p in enumerate(spec.inputs):
            t = torch.randn([int(x) for x in p.dims], generator=g)
            if spec.attrs.get("divide") and i == spec.attrs["den"]:
                t = t.abs() + 0.5      # denominators bounded away from zero, as the reference draws divisors
            inputs[p.name] = t.to(dt).to(device)
        vals = list(inputs.values())
        axes = spec.attrs["axes"]
        if spec.attrs.get("divide"):
            ni, di = spec.attrs["num"], spec.attrs["den"]
            outer = int(torch.tensor(vals[ni].shape[:axes[ni]]).prod()) if axes[ni] else 1
            num = vals[ni].float().sum(axes[ni]).reshape(outer, -1)
            den = vals[di].float().sum(axes[di]).reshape(outer, -1)   # one value per row, or one per element
            ref = num / den
        else:
            ref = vals[0].float().sum(axes[0])
        out = spec.outputs[0]
        return inputs, [ref.reshape([int(x) for x in out.dims]).to(dt)], graph_out_indices(spec)
    for p, base in zip(spec.inputs, spec.input_roles()):
        t = torch.randn([int(x) for x in p.dims], generator=g)
        if base == "w":
            t = t / d["K"] ** 0.5
        inputs[p.name] = by_role[base] = t.to(dt).to(device)
    S = spec.split
    if spec.family == "matmul":
        x, w = by_role["x"].float(), by_role["w"].float()
        kc = d["K"] // S
        ref = torch.stack([x[:, s * kc:(s + 1) * kc] @ w[s * kc:(s + 1) * kc] for s in range(S)])
        refs = [ref.reshape([int(v) for v in spec.outputs[0].dims]).to(dt)]
    elif spec.family == "attention_decode":
        q, k, v = (by_role[n].float() for n in ("q", "k", "v"))
        hq, hkv, skv, dd = d["HQ"], d["HKV"], d["SKV"], d["D"]
        scale, shift = float(spec.attrs.get("scale", dd ** -0.5)), float(spec.attrs.get("shift", 0.0))
        kk = k.repeat_interleave(hq // hkv, 0).view(hq, S, skv // S, dd)
        vv = v.repeat_interleave(hq // hkv, 0).view(hq, S, skv // S, dd)
        e = torch.exp(torch.einsum("hd,hstd->hst", q[:, 0], kk) * scale + shift)
        o_part, l_part = torch.einsum("hst,hstd->hsd", e, vv), e.sum(-1)
        refs = []
        for o in spec.outputs:
            src = o_part if int(torch.tensor([int(x) for x in o.dims]).prod()) == o_part.numel() else l_part
            refs.append(src.reshape([int(x) for x in o.dims]).to(dt))
    else:
        raise CompileError(f"{spec.family}: no two-stage form")
    del R
    return inputs, refs, graph_out_indices(spec)


def check_code(code_str, *, graph=None, dtype=None, out_idx=None, reference_cache_dir=None,
               tolerance: Tolerance | None = None, benchmark: BenchOptions | None = None):
    """``(kernel_source, latency_ms | None)``: load, bind, validate and optionally time one kernel.
    Picklable and top-level, so that spawned workers can run it (python/cleave/runtime/compile.py:151-173).
    ``graph`` and ``dtype`` are accepted for signature parity; the spec carries both."""
    with _stage("compile"):
        spec = _load_main_kernel_from_code(code_str)
        if out_idx is None:
            out_idx = graph_out_indices(spec)
        kernel = _compile(spec, out_idx)
    latency_ms = _check_kernel(kernel, spec=spec, reference_cache_dir=reference_cache_dir,
                               tolerance=tolerance or DEFAULT_TOLERANCE, benchmark=benchmark)
    return kernel.get_kernel_source(), latency_ms
