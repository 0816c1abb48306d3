"""The two kernel sets of the product: bfloat16 (serving) and float32 (true 32-bit).

Both drive the same hand-written launchers with a dtype code; they differ in the
element type of activations, weights and cache, and in the matrix products:

* bfloat16: products with float32 accumulation.  Plain ``x @ W.T`` goes to the
  library (cuBLAS through ``torch.mm``), as the reference's engine does for every
  product (worker/src/inference/qwen2/model.py:216-236); skinny and fused
  products use this package's own kernels where they are registered.
* float32: ``torch.mm`` with TF32 switched off, i.e. FMA-only float32 products;
  accurate ``expf``/``sincosf``/``rsqrtf`` in every kernel.

There is no CPU path here and no fallback: a missing library raises.
"""

from __future__ import annotations

import torch

import ctypes

from . import library
from .interface import KernelSet, StepTensors, Terms
from .library import KernelError, check, function

_CODE = {torch.float32: 0, torch.bfloat16: 1}
_DECODE_HEAD_DIMS = (16, 32, 64, 128, 256)
_PREFILL_HEAD_DIMS = (64, 128)  # tensor-core attention for portions of prompts (bfloat16)
_SKINNY_ROWS = 64               # weight-streaming products (tcgen05, weights as the 128-row operand) take up to 64 rows
_CLUSTER_SPLITS = 8             # splits of a decode attention that one cluster of CTAs merges itself
_TENSOR_CORE_ROWS = 128         # from here on the tcgen05 kernel's 128-row tiles are full; in between: the library
_MAX_TERMS = 24                 # terms of a pending sum that the layer-norm kernel adds up itself
_RULES = {"delta": 0, "ssd": 1, "gated": 2}
_GROUPED_TENSOR_CORE_PAIRS = 512  # (token, expert) pairs from which the routed products run on the tcgen05 tile kernel

_ERROR_TEXT = {
    1: "a token id outside the vocabulary reached the embedding",
    2: "a new token's page is missing from its block table (cache write)",
    3: "a block table does not cover the keys a token attends to",
    4: "a block table does not cover the keys a decoded token attends to",
    6: "a tensor-core product gave up waiting for its own copies or instructions",
    7: "a router chose an expert that does not exist",
    5: "a block table does not cover the keys a portion of a prompt attends to",
}


class DeviceKernels(KernelSet):
    def __init__(self, dtype: torch.dtype, device: torch.device | str = "cuda:0") -> None:
        if dtype not in _CODE:
            raise KernelError(f"no kernel set for dtype {dtype}; the engine runs bfloat16 or float32")
        self.dtype = dtype
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise KernelError("distie_b200 runs on a CUDA device (sm_100a) only; no GPU is visible")
        major, minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise KernelError(f"kernels are built for sm_100a; device reports sm_{major}{minor}")
        self.code = _CODE[dtype]
        if dtype == torch.float32:
            # True 32-bit products: no TF32, no reduced-precision reductions.
            torch.backends.cuda.matmul.allow_tf32 = False
            torch.backends.cudnn.allow_tf32 = False
            torch.set_float32_matmul_precision("highest")
        library.load_unit("base")
        if dtype == torch.bfloat16:
            library.load_unit("bf16")
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.launches = 0  # own kernels launched (library products are not counted)
        self.kernel_counts: dict[str, int] = {}  # the same, by launcher

    # -- helpers ------------------------------------------------------------
    @staticmethod
    def _stream() -> int:
        return torch.cuda.current_stream().cuda_stream

    def _ran(self, name: str, kernels: int = 1) -> None:
        self.launches += kernels
        self.kernel_counts[name] = self.kernel_counts.get(name, 0) + 1

    def check_errors(self) -> None:
        code = int(self.error_flag.item())
        if code:
            self.error_flag.zero_()
            raise KernelError(f"device-side check failed: {_ERROR_TEXT.get(code, code)}")

    # -- operations -----------------------------------------------------------
    def embed(self, step: StepTensors, table: torch.Tensor, residual: torch.Tensor) -> None:
        hidden = table.shape[1]
        check(
            function("distie_embed")(
                step.token_ids.data_ptr(), table.data_ptr(), residual.data_ptr(), step.num_tokens, hidden,
                table.shape[0], _CODE[table.dtype], self.error_flag.data_ptr(), self._stream(),
            ),
            "embed",
        )
        self._ran("embed")

    def add_rmsnorm(self, delta, residual, weight, eps, out, rows_index=None) -> None:
        rows = out.shape[0]
        rows_ptr = rows_index.data_ptr() if rows_index is not None else None
        if delta is not None and delta.dim() == 3:
            code = function("distie_add_rmsnorm_split")(
                delta.data_ptr(), delta.shape[0], delta.stride(0), residual.data_ptr(), weight.data_ptr(),
                out.data_ptr(), rows_ptr, rows, residual.shape[1], float(eps), self.code, self._stream(),
            )
            if code == 0:
                self._ran("add_rmsnorm_split")
                return
            if code != -2:
                check(code, "add_rmsnorm_split")
            # A width the fused kernel refuses: add the slices up here, in float32.
            summed = delta[0] if delta.shape[0] == 1 else delta.sum(0)
            if rows_index is None:
                residual.add_(summed)
                delta = None
            else:
                index = rows_index.long()
                residual, delta, rows_ptr = residual.index_select(0, index) + summed.index_select(0, index), None, None
        check(
            function("distie_add_rmsnorm")(
                delta.data_ptr() if delta is not None else None, residual.data_ptr(), weight.data_ptr(),
                out.data_ptr(), rows_ptr, rows, residual.shape[1], float(eps), self.code, self._stream(),
            ),
            "add_rmsnorm",
        )
        self._ran("add_rmsnorm")

    def linear_split(self, x, weight):
        if self._skinny(x, weight):
            m, n, k = x.shape[0], weight.shape[0], weight.shape[1]
            splits = function("distie_gemm_tcgen05_skinny_splits")(n, k, self.sm_count)
            out = torch.empty((splits, m, n), dtype=torch.float32, device=x.device)
            self._stream_weights(x, weight, None, out, 0)
            return out
        return super().linear_split(x, weight)

    def linear(self, x, weight, bias=None, out_dtype=None):
        out_dtype = out_dtype or self.dtype
        if weight.dtype == torch.float32:
            # float32 engine, or a matrix the checkpoint stores in 32-bit: a true float32 product.
            x32 = x if x.dtype == torch.float32 else x.float()
            y = torch.addmm(bias, x32, weight.t()) if bias is not None else torch.mm(x32, weight.t())
            return y if out_dtype == torch.float32 else self._bias_cast(y, None, out_dtype)
        if self._skinny(x, weight):
            out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=x.device)
            self._stream_weights(x, weight, bias, out, 1)
            return out
        if self._tensor_core(x, weight) and (bias is None or out_dtype == torch.float32) and not self._underfilled(x, weight):
            out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=x.device)
            self._gemm_tcgen05(x, weight, out, 1 if out_dtype == torch.float32 else 0)
            return out if bias is None else out.add_(bias)
        if bias is None and out_dtype == self.dtype:
            return torch.mm(x, weight.t())
        y32 = torch.mm(x, weight.t(), out_dtype=torch.float32)
        if out_dtype == torch.float32:
            return y32 if bias is None else y32.add_(bias)
        return self._bias_cast(y32, bias, out_dtype)

    def _tensor_core(self, x, weight) -> bool:
        """Products of more rows than the weight-streaming kernel takes: the tcgen05 kernel."""
        return (
            self.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
            and x.shape[0] >= _TENSOR_CORE_ROWS and weight.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and x.stride(1) == 1 and weight.is_contiguous()
        )

    def _underfilled(self, x, weight) -> bool:
        """A long-K product whose 256 x 256 tiles would leave most of the machine idle (a few hundred rows against
        a narrow weight, e.g. the down projection of a short portion): the library splits K over the idle SMs and
        is up to twice as fast there (measured at 256 to 1,024 rows of the 1.5B, 7B and 14B down projections)."""
        rows, n, k = x.shape[0], weight.shape[0], weight.shape[1]
        tiles = -(-rows // 256) * -(-n // 256)
        return k >= 4096 and tiles < 0.7 * (self.sm_count // 2)

    def _gemm_tcgen05(self, x, weight, out, epi: int, tile_width: int = 0) -> None:
        check(
            function("distie_gemm_tcgen05")(
                x.data_ptr(), x.stride(0), weight.data_ptr(), out.data_ptr(), out.stride(0), x.shape[0],
                weight.shape[0], weight.shape[1], epi, tile_width, self.sm_count, self.error_flag.data_ptr(),
                self._stream(),
            ),
            "gemm_tcgen05",
        )
        self._ran("gemm_tcgen05")

    def _skinny(self, x, weight) -> bool:
        return (
            self.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
            and x.shape[0] <= _SKINNY_ROWS and weight.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) == 1
            and weight.is_contiguous()
        )

    def _stream_weights(self, x, weight, bias, out, mode: int) -> None:
        """mode 0: float32 slices; 1: x W^T + bias; 2: fused SwiGLU (see gemm_tcgen05.cu)."""
        check(
            function("distie_gemm_tcgen05_skinny")(
                x.data_ptr(), x.stride(0), weight.data_ptr(), bias.data_ptr() if bias is not None else None,
                out.data_ptr(), out.stride(-2), x.shape[0], weight.shape[0], weight.shape[1], mode,
                _CODE.get(out.dtype, 0), self.sm_count, self.error_flag.data_ptr(), self._stream(),
            ),
            "gemm_tcgen05_skinny",
        )
        self._ran("gemm_tcgen05_skinny")

    def linear_swiglu(self, x, weight):
        if self._skinny(x, weight) and weight.shape[0] % 2 == 0:
            out = torch.empty((x.shape[0], weight.shape[0] // 2), dtype=self.dtype, device=x.device)
            self._stream_weights(x, weight, None, out, 2)
            return out
        if self._tensor_core(x, weight) and weight.shape[0] % 2 == 0:
            out = torch.empty((x.shape[0], weight.shape[0] // 2), dtype=self.dtype, device=x.device)
            self._gemm_tcgen05(x, weight, out, 2)
            return out
        return super().linear_swiglu(x, weight)

    def _bias_cast(self, y32, bias, out_dtype):
        out = torch.empty(y32.shape, dtype=out_dtype, device=y32.device)
        check(
            function("distie_bias_cast")(
                y32.data_ptr(), bias.data_ptr() if bias is not None else None, out.data_ptr(), y32.shape[0],
                y32.shape[1], _CODE[out_dtype], self._stream(),
            ),
            "bias_cast",
        )
        self._ran("bias_cast")
        return out

    def swiglu(self, gate_up, out) -> None:
        check(
            function("distie_swiglu")(
                gate_up.data_ptr(), out.data_ptr(), gate_up.shape[0], out.shape[1], self.code, self._stream()
            ),
            "swiglu",
        )
        self._ran("swiglu")

    def rope_kv_write(self, qkv, step, kv, rotary, num_heads, num_kv_heads, head_dim, bias=None, q_out=None) -> None:
        write = kv is not None
        table = kv.block_table if write else step.seq_seat  # any valid pointer when nothing is written
        tail = [
            step.positions.data_ptr(), step.token_seq.data_ptr(), step.seq_seat.data_ptr(),
            table.data_ptr(), table.shape[-1] if write else 1,
            rotary.inv_freq.data_ptr() if rotary is not None else None,
            float(rotary.factor) if rotary is not None else 1.0,
            kv.k.data_ptr() if write else None, kv.v.data_ptr() if write else None,
        ]
        sizes = [
            num_heads, num_kv_heads, head_dim,
            rotary.rotary_dim if rotary is not None else 0,
            int(rotary.interleaved) if rotary is not None else 0,
            kv.page_size if write else 1, kv.num_pages if write else 1, int(write), self.code,
            self.error_flag.data_ptr(), self._stream(),
        ]
        if qkv.dim() == 3:
            if q_out is None:
                raise KernelError("rope_kv_write: slices of a projection need a q_out buffer")
            code = function("distie_rope_kv_write_split")(
                qkv.data_ptr(), qkv.shape[0], qkv.stride(0), qkv.stride(1),
                bias.data_ptr() if bias is not None else None, q_out.data_ptr(), q_out.stride(0),
                *tail, step.num_tokens, *sizes,
            )
            if code == 0:
                self._ran("rope_kv_write_split")
                return
            if code != -2:
                check(code, "rope_kv_write_split")
            # Sizes the fused kernel refuses: finish the projection here, rotate in place, copy q out.
            summed = qkv[0] if qkv.shape[0] == 1 else qkv.sum(0)
            if bias is not None:
                summed = summed + bias
            dense = summed.to(self.dtype)
            self.rope_kv_write(dense, step, kv, rotary, num_heads, num_kv_heads, head_dim)
            q_out.copy_(dense[:, : num_heads * head_dim])
            return
        check(
            function("distie_rope_kv_write")(qkv.data_ptr(), *tail, step.num_tokens, qkv.stride(0), *sizes),
            "rope_kv_write",
        )
        self._ran("rope_kv_write")
        if q_out is not None:
            q_out.copy_(qkv[:, : num_heads * head_dim])

    def qkv_rope_write(self, x, weight, bias, step, kv, rotary, num_heads, num_kv_heads, head_dim, q_out) -> None:
        """Prompt portions of 128 rows and more: bias, rotation and the stores of q, k and v happen in the
        epilogue of the tcgen05 product, which reads the step's angles and cache rows from a table made once
        per step.  Everything else: the product's float32 slices into the rotation kernel."""
        fused = (
            self._tensor_core(x, weight) and head_dim in (64, 128)
            and weight.shape[0] == (num_heads + 2 * num_kv_heads) * head_dim
            and (rotary is None or (rotary.rotary_dim == head_dim and not rotary.interleaved))
            and (bias is None or bias.dtype == torch.float32)
            and (kv is None or kv.k.dtype == torch.bfloat16)
            and q_out.dtype == torch.bfloat16 and q_out.stride(1) == 1 and q_out.stride(0) % 8 == 0
            and not self._underfilled(x, weight)
        )
        if not fused:
            return super().qkv_rope_write(x, weight, bias, step, kv, rotary, num_heads, num_kv_heads, head_dim, q_out)
        trig, cache_row = self._rope_rows(step, kv, rotary, num_kv_heads, head_dim)
        check(
            function("distie_gemm_tcgen05_qkv")(
                x.data_ptr(), x.stride(0), weight.data_ptr(), bias.data_ptr() if bias is not None else None,
                trig.data_ptr(), cache_row.data_ptr() if cache_row is not None else None, q_out.data_ptr(),
                q_out.stride(0), kv.k.data_ptr() if kv is not None else None, kv.v.data_ptr() if kv is not None else None,
                x.shape[0], weight.shape[0], weight.shape[1], num_heads, num_kv_heads, head_dim,
                kv.page_size if kv is not None else 1, self.sm_count, self.error_flag.data_ptr(), self._stream(),
            ),
            "gemm_tcgen05_qkv",
        )
        self._ran("gemm_tcgen05_qkv")

    def _rope_rows(self, step, kv, rotary, num_kv_heads: int, head_dim: int):
        """(trig [T, head_dim] float32, cache_row [T] int32 or None) of this step: made by the first layer that
        asks and kept with the step for the others of its cache group and encoding."""
        key = (
            "rope_rows", head_dim, num_kv_heads, kv.block_table.data_ptr() if kv is not None else 0,
            rotary.inv_freq.data_ptr() if rotary is not None else 0, float(rotary.factor) if rotary is not None else 1.0,
        )
        made = step.derived.get(key)
        if made is None:
            trig = torch.empty((step.num_tokens, head_dim), dtype=torch.float32, device=self.device)
            cache_row = torch.empty(step.num_tokens, dtype=torch.int32, device=self.device) if kv is not None else None
            check(
                function("distie_rope_rows")(
                    step.positions.data_ptr(), step.token_seq.data_ptr(), step.seq_seat.data_ptr(),
                    kv.block_table.data_ptr() if kv is not None else None, kv.block_table.shape[-1] if kv is not None else 1,
                    rotary.inv_freq.data_ptr() if rotary is not None else None,
                    float(rotary.factor) if rotary is not None else 1.0, step.num_tokens, head_dim, num_kv_heads,
                    kv.page_size if kv is not None else 1, kv.num_pages if kv is not None else 1, trig.data_ptr(),
                    cache_row.data_ptr() if cache_row is not None else None, self.error_flag.data_ptr(), self._stream(),
                ),
                "rope_rows",
            )
            self._ran("rope_rows")
            made = step.derived[key] = (trig, cache_row)
        return made

    def plan_splits(self, tokens: int, num_heads: int, num_kv_heads: int, max_kv_len: int) -> int:
        group = num_heads // num_kv_heads
        chunks = (group + 7) // 8 if group > 8 else 1
        blocks = max(1, tokens * num_kv_heads * chunks)
        by_machine = max(1, 2 * self.sm_count // blocks)  # two CTAs fit an SM; a second wave would wait for the first
        by_length = max(1, max_kv_len // 256)
        return max(1, min(by_machine, by_length, 64))

    def qkv_attention(self, x, weight, bias, step, kv, writes_cache, rotary, num_heads, num_kv_heads, head_dim,
                      window, scale, out, chunk=None) -> None:
        """A step of single tokens on the tensor-core kernels: the attention kernel starts from the
        projection's float32 slices itself (bias, rotation, the token's key and value into the cache and into
        its own tile), so the kernel between the projection and the attention is not launched."""
        merged = (
            step.num_decode_tokens == step.num_tokens and self.dtype == torch.bfloat16 and head_dim in _PREFILL_HEAD_DIMS
            and self._skinny(x, weight) and weight.shape[0] == (num_heads + 2 * num_kv_heads) * head_dim
            and (rotary is None or (rotary.rotary_dim == head_dim and not rotary.interleaved))
            and (bias is None or bias.dtype == torch.float32) and kv.k.dtype == torch.bfloat16
            and out.dtype == torch.bfloat16
        )
        if not merged:
            return super().qkv_attention(x, weight, bias, step, kv, writes_cache, rotary, num_heads, num_kv_heads,
                                         head_dim, window, scale, out, chunk)
        slices = self.linear_split(x, weight)
        window = int(window) if window else 0
        chunk = int(chunk) if chunk else 0
        tokens = step.num_tokens
        splits = self.plan_splits(tokens, num_heads, num_kv_heads, step.max_kv_len)
        if splits <= 2 * _CLUSTER_SPLITS:
            splits = min(splits, _CLUSTER_SPLITS)  # merged inside the kernel, by a cluster of CTAs
        scratch = None
        if splits > _CLUSTER_SPLITS:
            floats = function("distie_attention_decode_scratch_floats")(tokens, num_heads, head_dim, splits)
            scratch = torch.empty(floats, dtype=torch.float32, device=x.device)
        check(
            function("distie_attention_decode_mma_qkv")(
                slices.data_ptr(), slices.shape[0], slices.stride(0), slices.stride(1),
                bias.data_ptr() if bias is not None else None,
                rotary.inv_freq.data_ptr() if rotary is not None else None,
                float(rotary.factor) if rotary is not None else 1.0, int(bool(writes_cache)),
                out.data_ptr(), out.stride(0), scratch.data_ptr() if scratch is not None else None,
                step.positions.data_ptr(), step.token_seq.data_ptr(), step.seq_seat.data_ptr(),
                kv.block_table.data_ptr(), kv.block_table.shape[-1], kv.k.data_ptr(), kv.v.data_ptr(), tokens,
                num_heads, num_kv_heads, head_dim, kv.page_size, kv.num_pages, window, chunk, float(scale), splits,
                self.error_flag.data_ptr(), self._stream(),
            ),
            "attention_decode_mma_qkv",
        )
        self._ran("attention_decode_mma", 1 if splits <= _CLUSTER_SPLITS else 2)
        self._ran("attention_decode_mma_qkv", 0)

    def attention(self, qkv, out, step, kv, num_heads, num_kv_heads, head_dim, window, scale, chunk=None,
                  keep_first=0, softcap=0.0, sink=None) -> None:
        window = int(window) if window else 0
        chunk = int(chunk) if chunk else 0
        keep_first = int(keep_first) if keep_first and window else 0
        softcap = float(softcap or 0.0)
        sink_ptr = sink.data_ptr() if sink is not None else None
        if sink is not None and (sink.dtype != torch.float32 or sink.numel() != num_heads or not sink.is_contiguous()):
            raise KernelError("attention: the sink is one float32 per head")
        extras = softcap > 0.0 or sink is not None
        value_dim = kv.v.shape[-1]
        same = value_dim == head_dim  # every kernel but the size-agnostic one wants values as large as keys
        n_dec = step.num_decode_tokens if head_dim in _DECODE_HEAD_DIMS and same else 0
        element = qkv.element_size()
        if n_dec > 0:
            splits = self.plan_splits(n_dec, num_heads, num_kv_heads, step.max_kv_len)
            tensor_cores = self.dtype == torch.bfloat16 and head_dim in _PREFILL_HEAD_DIMS
            if tensor_cores and splits <= 2 * _CLUSTER_SPLITS:
                splits = min(splits, _CLUSTER_SPLITS)  # merged inside the kernel, by a cluster of CTAs
            in_kernel_merge = splits == 1 or (tensor_cores and splits <= _CLUSTER_SPLITS)
            scratch = None
            if not in_kernel_merge:
                floats = function("distie_attention_decode_scratch_floats")(n_dec, num_heads, head_dim, splits)
                scratch = torch.empty(floats, dtype=torch.float32, device=qkv.device)
            head = [
                qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0),
                scratch.data_ptr() if scratch is not None else None, step.positions.data_ptr(),
                step.token_seq.data_ptr(), step.seq_seat.data_ptr(), kv.block_table.data_ptr(),
                kv.block_table.shape[-1], kv.k.data_ptr(), kv.v.data_ptr(), n_dec, num_heads, num_kv_heads,
                head_dim, kv.page_size, kv.num_pages, window, chunk,
            ]
            if tensor_cores and extras:
                check(
                    function("distie_attention_decode_mma_capped")(*head, keep_first, float(scale), softcap, sink_ptr, splits,
                                                                   self.error_flag.data_ptr(), self._stream()),
                    "attention_decode_mma",
                )
            elif tensor_cores:
                check(
                    function("distie_attention_decode_mma_kept")(*head, keep_first, float(scale), splits,
                                                                 self.error_flag.data_ptr(), self._stream()),
                    "attention_decode_mma",
                )
            else:
                check(
                    function("distie_attention_decode_capped")(*head, keep_first, float(scale), softcap, sink_ptr, splits, self.code,
                                                        self.error_flag.data_ptr(), self._stream()),
                    "attention_decode",
                )
            self._ran("attention_decode_mma" if tensor_cores else "attention_decode", 1 if in_kernel_merge else 2)
        rest = step.num_tokens - n_dec
        tiled = (rest > 0 and self.dtype == torch.bfloat16 and head_dim in _PREFILL_HEAD_DIMS and step.num_q_tiles
                 and n_dec == step.num_decode_tokens and same)
        if tiled and self._attention_tcgen05(qkv, out, step, kv, num_heads, num_kv_heads, head_dim, window, chunk, scale,
                                             keep_first, softcap, sink_ptr):
            pass
        elif tiled:
            check(
                function("distie_attention_prefill")(
                    qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), step.q_tiles.data_ptr(),
                    step.num_q_tiles, step.positions.data_ptr(), step.token_seq.data_ptr(), step.seq_seat.data_ptr(),
                    kv.block_table.data_ptr(), kv.block_table.shape[-1], kv.k.data_ptr(), kv.v.data_ptr(), num_heads,
                    num_kv_heads, head_dim, kv.page_size, kv.num_pages, window, chunk, keep_first, float(scale),
                    softcap, sink_ptr, self.error_flag.data_ptr(), self._stream(),
                ),
                "attention_prefill",
            )
            self._ran("attention_prefill")
        elif rest > 0:
            check(
                function("distie_attention_generic")(
                    qkv.data_ptr() + n_dec * qkv.stride(0) * element, qkv.stride(0),
                    out.data_ptr() + n_dec * out.stride(0) * element, out.stride(0),
                    step.positions.data_ptr() + 4 * n_dec, step.token_seq.data_ptr() + 4 * n_dec,
                    step.seq_seat.data_ptr(), kv.block_table.data_ptr(), kv.block_table.shape[-1],
                    kv.k.data_ptr(), kv.v.data_ptr(), rest, num_heads, num_kv_heads, head_dim, value_dim, kv.page_size,
                    kv.num_pages, window, chunk, keep_first, float(scale), softcap, sink_ptr, self.code,
                    self.error_flag.data_ptr(), self._stream(),
                ),
                "attention_generic",
            )
            self._ran("attention_generic")

    def _attention_tcgen05(self, qkv, out, step, kv, num_heads, num_kv_heads, head_dim, window, chunk, scale,
                           keep_first=0, softcap=0.0, sink_ptr=None) -> bool:
        """Prompt portions on the tcgen05 kernel; False when it refuses the page size or an alignment."""
        code = function("distie_attention_prefill_tcgen05")(
            qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), step.q_tiles.data_ptr(), step.num_q_tiles,
            step.positions.data_ptr(), step.token_seq.data_ptr(), step.seq_seat.data_ptr(),
            kv.block_table.data_ptr(), kv.block_table.shape[-1], kv.k.data_ptr(), kv.v.data_ptr(), qkv.shape[0],
            num_heads, num_kv_heads, head_dim, kv.page_size, kv.num_pages, window, chunk, keep_first, float(scale),
            float(softcap), sink_ptr, self.error_flag.data_ptr(), self._stream(),
        )
        if code == -2:
            return False
        check(code, "attention_prefill_tcgen05")
        self._ran("attention_prefill_tcgen05")
        return True

    # -- layers with per-request state: layer norm over a pending sum, gates, convolutions, recurrences ---------
    def add_layernorm(self, delta, residual, weight, bias, eps, out, rows_index=None) -> None:
        pairs = [] if delta is None else Terms.of(delta).flat()
        if len(pairs) > _MAX_TERMS:  # more terms than the kernel takes: the tail is summed here, in float32
            tail = Terms(pairs[_MAX_TERMS - 1 :]).total()
            pairs = pairs[: _MAX_TERMS - 1] + [(tail, 1.0)]
        pairs = [(t if t.is_contiguous() else t.contiguous(), s) for t, s in pairs]
        pointers = (ctypes.c_void_p * max(1, len(pairs)))(*[t.data_ptr() for t, _ in pairs])
        scales = (ctypes.c_float * max(1, len(pairs)))(*[s for _, s in pairs])
        check(
            function("distie_add_layernorm")(
                pointers, scales, len(pairs), residual.data_ptr(), weight.data_ptr(), bias.data_ptr(), out.data_ptr(),
                rows_index.data_ptr() if rows_index is not None else None, out.shape[0], residual.shape[1], float(eps),
                self.code, self._stream(),
            ),
            "add_layernorm",
        )
        self._ran("add_layernorm")

    @staticmethod
    def _rows32(x: torch.Tensor, what: str) -> torch.Tensor:
        if x.dtype != torch.float32 or x.stride(-1) != 1:
            raise KernelError(f"{what}: a float32 matrix with unit column stride is expected")
        return x

    @classmethod
    def _sliced(cls, x: torch.Tensor, what: str) -> tuple[int, int, int, int]:
        """(pointer, row stride, slices, slice stride) of a float32 matrix or of the slices ``[S, T, n]`` it is the sum of."""
        cls._rows32(x, what)
        if x.dim() == 3:
            return x.data_ptr(), x.stride(1), x.shape[0], x.stride(0)
        return x.data_ptr(), x.stride(0), 1, 0

    def kv_write(self, k, v, step, kv) -> None:
        if k.dtype != v.dtype or k.dtype not in _CODE or k.stride(1) != 1 or v.stride(1) != 1:
            raise KernelError("kv_write: keys and values of one float type with unit column stride are expected")
        check(
            function("distie_kv_write")(
                k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), _CODE[k.dtype], step.positions.data_ptr(),
                step.token_seq.data_ptr(), step.seq_seat.data_ptr(), kv.block_table.data_ptr(), kv.block_table.shape[-1],
                kv.k.data_ptr(), kv.v.data_ptr(), step.num_tokens, kv.k.shape[1], kv.k.shape[-1], kv.v.shape[-1],
                kv.page_size, kv.num_pages, _CODE[kv.k.dtype], self.error_flag.data_ptr(), self._stream(),
            ),
            "kv_write",
        )
        self._ran("kv_write")

    def head_gate(self, x, logits, num_heads) -> None:
        if not x.is_contiguous():
            raise KernelError("head_gate: a contiguous activation is expected")
        check(
            function("distie_head_gate")(
                x.data_ptr(), *self._sliced(logits, "head_gate"), x.shape[0], num_heads, x.shape[1] // num_heads,
                _CODE[x.dtype], self._stream(),
            ),
            "head_gate",
        )
        self._ran("head_gate")

    def prepare_step(self, step) -> None:
        """What several sublayers of a block share of the step, made before they part onto streams of their own."""
        self._seq_index(step)

    def _seq_index(self, step):
        """(token_first [T], seq_bounds [B + 1]), int32: where each token's request starts among the step's tokens and
        the range of every batch row; made once per step on the device and kept with it for all layers."""
        made = step.derived.get("seq_index")
        if made is None:
            both = torch.empty(step.num_tokens + step.num_seqs + 1, dtype=torch.int32, device=self.device)
            token_first, bounds = both[: step.num_tokens], both[step.num_tokens :]
            check(
                function("distie_seq_index")(step.token_seq.data_ptr(), step.num_tokens, step.num_seqs,
                                             token_first.data_ptr(), bounds.data_ptr(), self._stream()),
                "seq_index",
            )
            self._ran("seq_index")
            made = step.derived["seq_index"] = (token_first, bounds)
        return made

    def short_conv(self, x, weight, bias, state, step, activation="silu", input_bias=None):
        sliced = self._sliced(x, "short_conv")
        channels, taps = weight.shape
        out = torch.empty((step.num_tokens, channels), dtype=torch.float32, device=x.device)
        single = step.num_decode_tokens == step.num_tokens  # one token per request: the kernel moves the state on itself
        token_first, seq_bounds = self._seq_index(step)
        check(
            function("distie_short_conv")(
                *sliced, weight.data_ptr(), bias.data_ptr() if bias is not None else None,
                state.data_ptr() if state is not None else None, step.token_seq.data_ptr(), token_first.data_ptr(),
                seq_bounds.data_ptr(), step.seq_seat.data_ptr(), step.num_tokens, step.num_seqs, channels, taps, int(activation == "silu"), int(single), out.data_ptr(),
                input_bias.data_ptr() if input_bias is not None else None, self._stream(),
            ),
            "short_conv",
        )
        self._ran("short_conv", 2 if taps > 1 and not single else 1)
        return out

    def linear_recurrence(self, rule, q, k, v, decay, write, state, step, heads, groups, key_dim, value_dim,
                          decay_rate=None, decay_bias=None, skip=None, unit_column=False):
        for name, t in (("q", q), ("k", k), ("v", v)):
            self._rows32(t, f"linear_recurrence {name}")
        none = (None, 0, 1, 0)
        decay_ptr, decay_stride, splits, split_stride = self._sliced(decay, "linear_recurrence decay") if decay is not None else none
        write_ptr, write_stride, write_splits, write_split_stride = (
            self._sliced(write, "linear_recurrence write") if write is not None else (None, 0, splits, split_stride))
        if decay is None:
            splits, split_stride = write_splits, write_split_stride
        if (splits, split_stride) != (write_splits, write_split_stride):
            raise KernelError("linear_recurrence: decay and write are views of one projection")
        out = torch.empty((step.num_tokens, heads * value_dim), dtype=torch.float32, device=q.device)
        scratch = torch.empty(step.num_tokens * (2 * heads + groups), dtype=torch.float32, device=q.device)
        check(
            function("distie_linear_recurrence")(
                _RULES[rule], q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
                decay_ptr, decay_stride, write_ptr, write_stride, splits, split_stride,
                decay_rate.data_ptr() if decay_rate is not None else None,
                decay_bias.data_ptr() if decay_bias is not None else None, skip.data_ptr() if skip is not None else None,
                state.data_ptr(), out.data_ptr(), out.stride(0), scratch.data_ptr(), self._seq_index(step)[1].data_ptr(),
                step.seq_seat.data_ptr(), step.num_tokens, step.num_seqs, heads, groups, key_dim, value_dim,
                int(bool(unit_column)), self._stream(),
            ),
            "linear_recurrence",
        )
        self._ran("linear_recurrence", 2)
        return out

    def gated_rmsnorm(self, x, gate, weight, eps, group, gate_first, out, activation="silu") -> None:
        self._rows32(x, "gated_rmsnorm x")
        check(
            function("distie_gated_rmsnorm")(
                x.data_ptr(), x.stride(0), *self._sliced(gate, "gated_rmsnorm gate"), weight.data_ptr(), weight.numel(),
                out.data_ptr(), out.stride(0), x.shape[0], x.shape[1], group, float(eps),
                int(bool(gate_first)) | (2 if activation == "sigmoid" else 0),
                _CODE[out.dtype], self._stream(),
            ),
            "gated_rmsnorm",
        )
        self._ran("gated_rmsnorm")

    # -- norms around a sublayer, keys as values, memories with exponential gates, routed feed-forwards -------------
    def norm_add_rmsnorm(self, delta, delta_weight, delta_eps, residual, weight, eps, out, rows_index=None) -> None:
        pairs = [] if delta is None else Terms.of(delta).flat()
        if len(pairs) > _MAX_TERMS:  # more terms than the kernel takes: the tail is summed here, in float32
            tail = Terms(pairs[_MAX_TERMS - 1 :]).total()
            pairs = pairs[: _MAX_TERMS - 1] + [(tail, 1.0)]
        pairs = [(t if t.is_contiguous() else t.contiguous(), s) for t, s in pairs]
        pointers = (ctypes.c_void_p * max(1, len(pairs)))(*[t.data_ptr() for t, _ in pairs])
        scales = (ctypes.c_float * max(1, len(pairs)))(*[s for _, s in pairs])
        rows = out.shape[0] if out is not None else residual.shape[0]
        check(
            function("distie_norm_add_rmsnorm")(
                pointers, scales, len(pairs), delta_weight.data_ptr() if delta_weight is not None else None,
                float(delta_eps), residual.data_ptr(), weight.data_ptr() if weight is not None else None, float(eps),
                out.data_ptr() if out is not None else None, rows_index.data_ptr() if rows_index is not None else None,
                rows, residual.shape[1], _CODE[out.dtype] if out is not None else self.code, self._stream(),
            ),
            "norm_add_rmsnorm",
        )
        self._ran("norm_add_rmsnorm")

    def qk_rope_norm_write(self, qk, bias, step, kv, rotary, num_heads, num_kv_heads, head_dim, norm_eps, q_out) -> None:
        write = kv is not None
        if write and kv.k.dtype != q_out.dtype:
            raise KernelError("qk_rope_norm_write: the cache and q are of one type")
        table = kv.block_table if write else step.seq_seat
        check(
            function("distie_qk_rope_norm_write")(
                *self._sliced(qk, "qk_rope_norm_write"), bias.data_ptr() if bias is not None else None, q_out.data_ptr(),
                q_out.stride(0), step.positions.data_ptr(), step.token_seq.data_ptr(), step.seq_seat.data_ptr(),
                table.data_ptr(), table.shape[-1] if write else 1,
                rotary.inv_freq.data_ptr() if rotary is not None else None,
                float(rotary.factor) if rotary is not None else 1.0, kv.k.data_ptr() if write else None,
                kv.v.data_ptr() if write else None, step.num_tokens, num_heads, num_kv_heads, head_dim,
                rotary.rotary_dim if rotary is not None else 0, int(rotary.interleaved) if rotary is not None else 0,
                kv.page_size if write else 1, kv.num_pages if write else 1, int(write), int(norm_eps is not None),
                float(norm_eps or 0.0), _CODE[q_out.dtype], self.error_flag.data_ptr(), self._stream(),
            ),
            "qk_rope_norm_write",
        )
        self._ran("qk_rope_norm_write")

    def qkv_norm_write(self, qkv, bias, step, kv, rotary, num_heads, num_kv_heads, head_dim, value_dim, norm_eps,
                       q_weight, k_weight, q_temp, q_out) -> None:
        write = kv is not None
        if write and (kv.k.dtype != q_out.dtype or kv.v.shape[-1] != value_dim or kv.k.shape[-1] != head_dim):
            raise KernelError("qkv_norm_write: the cache holds keys of head_dim and values of value_dim, of q's type")
        table = kv.block_table if write else step.seq_seat
        coef, every = (float(q_temp[0]), float(q_temp[1])) if q_temp else (0.0, 0.0)
        check(
            function("distie_qkv_norm_write")(
                *self._sliced(qkv, "qkv_norm_write"), bias.data_ptr() if bias is not None else None, q_out.data_ptr(),
                q_out.stride(0), step.positions.data_ptr(), step.token_seq.data_ptr(), step.seq_seat.data_ptr(),
                table.data_ptr(), table.shape[-1] if write else 1,
                rotary.inv_freq.data_ptr() if rotary is not None else None,
                float(rotary.factor) if rotary is not None else 1.0, kv.k.data_ptr() if write else None,
                kv.v.data_ptr() if write else None, step.num_tokens, num_heads, num_kv_heads, head_dim, value_dim,
                rotary.rotary_dim if rotary is not None else 0, int(rotary.interleaved) if rotary is not None else 0,
                kv.page_size if write else 1, kv.num_pages if write else 1, int(write), int(norm_eps is not None),
                float(norm_eps or 0.0), q_weight.data_ptr() if q_weight is not None else None,
                k_weight.data_ptr() if k_weight is not None else None, coef, every, _CODE[q_out.dtype],
                self.error_flag.data_ptr(), self._stream(),
            ),
            "qkv_norm_write",
        )
        self._ran("qkv_norm_write")

    def activation(self, x, kind="silu", scale=1.0, scaled_columns=0):
        if kind not in ("silu", "none"):
            raise KernelError(f"activation {kind!r}: 'silu' or 'none'")
        out = torch.empty((x.shape[-2], x.shape[-1]), dtype=torch.float32, device=x.device)
        check(
            function("distie_activation")(*self._sliced(x, "activation"), out.data_ptr(), out.shape[0], out.shape[1],
                                          int(kind == "silu"), float(scale), int(scaled_columns), self._stream()),
            "activation",
        )
        self._ran("activation")
        return out

    def exp_gate_scan(self, log_in, log_forget, in_bias, forget_bias, cap, state, step):
        in_ptr, stride, splits, split_stride = self._sliced(log_in, "exp_gate_scan input gate")
        forget_ptr, forget_stride, forget_splits, forget_split_stride = self._sliced(log_forget, "exp_gate_scan forget gate")
        if (stride, splits, split_stride) != (forget_stride, forget_splits, forget_split_stride):
            raise KernelError("exp_gate_scan: the two gates are views of one projection")
        heads = log_in.shape[-1]
        gates = torch.empty((3, step.num_tokens, heads), dtype=torch.float32, device=self.device)
        check(
            function("distie_exp_gate_scan")(
                in_ptr, forget_ptr, stride, splits, split_stride, in_bias.data_ptr(), forget_bias.data_ptr(), float(cap),
                state.data_ptr(), self._seq_index(step)[1].data_ptr(), step.seq_seat.data_ptr(), step.num_seqs,
                step.num_tokens, heads, gates[0].data_ptr(), gates[1].data_ptr(), gates[2].data_ptr(), self._stream(),
            ),
            "exp_gate_scan",
        )
        self._ran("exp_gate_scan", 3)
        return gates[0], gates[1], gates[2]

    def stabilized_readout(self, read, floor, heads, value_dim):
        self._rows32(read, "stabilized_readout")
        if not floor.is_contiguous():
            raise KernelError("stabilized_readout: a contiguous floor is expected")
        out = torch.empty((read.shape[0], heads * value_dim), dtype=torch.float32, device=read.device)
        check(
            function("distie_stabilized_readout")(read.data_ptr(), read.stride(0), floor.data_ptr(), out.data_ptr(),
                                                  read.shape[0], heads, value_dim, self._stream()),
            "stabilized_readout",
        )
        self._ran("stabilized_readout")
        return out

    def route_top(self, x, router, top, scoring="sigmoid", groups=None, weight_scale=1.0, extra_rows=0, correction=None,
                  normalise=False):
        if scoring not in ("sigmoid", "softmax"):
            raise KernelError(f"route_top: scoring {scoring!r} is not built; 'sigmoid' and 'softmax' are")
        softmax, norm = int(scoring == "softmax"), int(bool(normalise))
        correction_ptr = correction.data_ptr() if correction is not None else None
        library.load_unit("routed")
        if x.dtype != router.dtype:
            x = x.to(router.dtype)  # a router kept in 32-bit reads the activations widened
        if x.stride(1) != 1 or not router.is_contiguous():
            raise KernelError("route_top: rows with unit column stride are expected")
        extra = int(extra_rows)
        tokens, experts = x.shape[0], router.shape[0] - extra
        count, keep = (int(groups[0]), int(groups[1])) if groups is not None else (1, 1)
        ids = torch.empty((tokens, top), dtype=torch.int32, device=x.device)
        weights = torch.empty((tokens, top), dtype=torch.float32, device=x.device)
        if self._tensor_core(x, router):
            # Prompt portions in bfloat16: the logits are a product on the tcgen05 tile kernel (float32 accumulators,
            # stored as float32), and a small kernel picks from them.
            logits = torch.empty((tokens, experts + extra), dtype=torch.float32, device=x.device)
            self._gemm_tcgen05(x, router, logits, 1)
            check(function("distie_route_pick")(logits.data_ptr(), logits.stride(0), tokens, experts, top, ids.data_ptr(),
                                                weights.data_ptr(), count, keep, float(weight_scale), softmax, correction_ptr,
                                                norm, self._stream()),
                  "route_pick")
            self._ran("route_top")
            return (ids, weights, logits[:, experts:]) if extra else (ids, weights)
        extra_out = torch.empty((tokens, extra), dtype=torch.float32, device=x.device) if extra else None
        check(
            function("distie_route_top")(x.data_ptr(), x.stride(0), router.data_ptr(), tokens, x.shape[1], experts, top,
                                         ids.data_ptr(), weights.data_ptr(), count, keep, float(weight_scale), extra,
                                         extra_out.data_ptr() if extra else None, softmax, correction_ptr, norm,
                                         _CODE[x.dtype], self._stream()),
            "route_top",
        )
        self._ran("route_top")
        return (ids, weights, extra_out) if extra else (ids, weights)

    def routed_swiglu(self, x, ids, weights, gate_up, down, scale_input=True, limit=None, identity=0):
        identity = int(identity or 0)
        if identity and scale_input:
            raise KernelError("routed_swiglu: experts that return their input go with the weight on the output")
        if gate_up.dtype != x.dtype or down.dtype != x.dtype:
            if gate_up.dtype != down.dtype:
                raise KernelError("routed_swiglu: the experts' matrices are of one type")
            x = x.to(gate_up.dtype)
        if x.stride(1) != 1 or not gate_up.is_contiguous() or not down.is_contiguous():
            raise KernelError("routed_swiglu: contiguous expert matrices and rows with unit column stride are expected")
        tokens, top = ids.shape
        experts, hidden, ff = gate_up.shape[0], x.shape[1], down.shape[2]
        code = _CODE[x.dtype]
        if code == 1 and (x.stride(0) % 8 or hidden % 8 or ff % 8):
            # rows that are no multiples of 16 bytes: the float32 form of the grouped products takes any size
            x, gate_up, down, code = x.float(), gate_up.float(), down.float(), 0
        if code == 1 and self.dtype == torch.bfloat16 and tokens * top >= _GROUPED_TENSOR_CORE_PAIRS:
            return self._routed_swiglu_tcgen05(x, ids, weights, gate_up, down, scale_input, limit, identity)
        tile = function("distie_routed_tile")(code, hidden, ff, tokens * top, experts)
        words = function("distie_route_plan_words")(tokens * top, experts, tile)
        plan = torch.empty(words, dtype=torch.int32, device=x.device)
        mid = torch.empty((tokens * top, ff), dtype=x.dtype, device=x.device)
        out = torch.empty((top, tokens, hidden), dtype=torch.float32, device=x.device)
        check(
            function("distie_routed_swiglu")(
                x.data_ptr(), x.stride(0), ids.data_ptr(), weights.data_ptr(), gate_up.data_ptr(), down.data_ptr(),
                plan.data_ptr(), mid.data_ptr(), out.data_ptr(), tokens, top, experts, hidden, ff, int(bool(scale_input)),
                float(limit) if limit is not None else 0.0, identity, code, self.error_flag.data_ptr(), self._stream(),
            ),
            "routed_swiglu",
        )
        self._ran("routed_swiglu", 3)
        return out

    def _routed_swiglu_tcgen05(self, x, ids, weights, gate_up, down, scale_input, limit=None, identity=0):
        """Prompt portions in bfloat16: the rows sorted by expert (and scaled by their weights) are gathered once, and
        both products run on the tcgen05 tile kernel over a list of row tiles that stays on the device."""
        tokens, top = ids.shape
        experts, hidden, ff = gate_up.shape[0], x.shape[1], down.shape[2]
        pairs, tile = tokens * top, 128
        max_tiles = (pairs + tile - 1) // tile + experts
        words = function("distie_route_plan_words")(pairs, experts, tile)
        plan = torch.empty(words, dtype=torch.int32, device=x.device)
        base = plan.data_ptr()
        tile_expert, tile_first, tile_rows = (base + 4 * (1 + experts + 1 + i * max_tiles) for i in range(3))
        stream, error = self._stream(), self.error_flag.data_ptr()
        check(function("distie_route_plan")(ids.data_ptr(), weights.data_ptr(), tokens, top, experts, tile, base, error, identity,
                                            stream), "route_plan")
        gathered = torch.empty((pairs, hidden), dtype=x.dtype, device=x.device)
        check(function("distie_routed_gather")(x.data_ptr(), x.stride(0), base, pairs, experts, tile, gathered.data_ptr(), hidden,
                                               int(bool(scale_input)), 1, stream), "routed_gather")
        mid = torch.empty((pairs, ff), dtype=x.dtype, device=x.device)
        check(function("distie_gemm_tcgen05_grouped")(
            gathered.data_ptr(), hidden, pairs, gate_up.data_ptr(), experts, 2 * ff, mid.data_ptr(), ff, ff, hidden, 2,
            float(limit) if limit is not None else 0.0, base,
            tile_expert, tile_first, tile_rows, max_tiles, self.sm_count, error, stream), "gemm_tcgen05_grouped")
        sorted_out = torch.empty((pairs, hidden), dtype=torch.float32, device=x.device)
        check(function("distie_gemm_tcgen05_grouped")(
            mid.data_ptr(), ff, pairs, down.data_ptr(), experts, hidden, sorted_out.data_ptr(), hidden, hidden, ff, 1, 0.0, base,
            tile_expert, tile_first, tile_rows, max_tiles, self.sm_count, error, stream), "gemm_tcgen05_grouped")
        out = torch.empty((top, tokens, hidden), dtype=torch.float32, device=x.device)
        if identity:
            check(function("distie_routed_identity")(x.data_ptr(), x.stride(0), ids.data_ptr(), weights.data_ptr(), tokens, top,
                                                     experts, out.data_ptr(), hidden, _CODE[x.dtype], stream), "routed_identity")
        check(function("distie_routed_scatter")(sorted_out.data_ptr(), base, pairs, experts, tile, out.data_ptr(), hidden,
                                                int(not scale_input), stream), "routed_scatter")
        self._ran("routed_swiglu", 5)
        self._ran("gemm_tcgen05_grouped", 0)
        return out

    # -- gated and squared-ReLU hidden layers on float32 accumulators; attention through a latent ------------------
    def _glu_act(self, x32, ff: int, kind: int, limit, row_gate):
        library.load_unit("latent")
        tokens = x32.shape[-2]
        out = torch.empty((tokens, ff), dtype=self.dtype, device=x32.device)
        gate = self._sliced(row_gate, "glu_act") if row_gate is not None else (None, 0, 1, 0)
        check(
            function("distie_glu_act")(*self._sliced(x32, "glu_act"), tokens, ff, kind, float(limit) if limit is not None else 0.0,
                                       *gate, out.data_ptr(), out.stride(0), self.code, self._stream()),
            "glu_act",
        )
        self._ran("glu_act")
        return out

    def linear_glu(self, x, weight, limit=None, row_gate=None):
        if weight.shape[0] % 2:
            raise KernelError("linear_glu: gate rows and up rows are stacked, so the weight has an even number of rows")
        if limit is None and row_gate is None:
            return self.linear_swiglu(x, weight)
        if row_gate is not None and row_gate.dim() == 2 and row_gate.shape[-1] != 1:
            raise KernelError("linear_glu: the row gate is one logit per row")
        return self._glu_act(self.linear_split(x, weight), weight.shape[0] // 2, 0, limit, row_gate)

    def linear_act(self, x, weight, kind="relu2"):
        if kind != "relu2":
            raise KernelError(f"linear_act: activation {kind!r} is not built; 'relu2' is")
        return self._glu_act(self.linear_split(x, weight), weight.shape[0], 1, None, None)

    def latent_kv_write(self, proj, step, kv, rotary, q_rank, q_norm, kv_rank, kv_norm, rot_dim, eps, q_latent_out) -> None:
        library.load_unit("latent")
        write = kv is not None
        if write and (kv.k.dtype != q_latent_out.dtype or kv.k.shape[-1] != kv_rank + rot_dim or kv.k.shape[-3] != 1
                      or not kv.k.is_contiguous()):
            raise KernelError("latent_kv_write: the cache holds one contiguous row [kv_rank + rot_dim] per token, of q's type")
        table = kv.block_table if write else step.seq_seat
        turned = rotary.rotary_dim if rotary is not None else 0
        check(
            function("distie_latent_kv_write")(
                *self._sliced(proj, "latent_kv_write"), q_rank, q_norm.data_ptr(), kv_rank,
                kv_norm.data_ptr() if write else None, rot_dim, float(eps), q_latent_out.data_ptr(), q_latent_out.stride(0),
                step.positions.data_ptr(), step.token_seq.data_ptr(), step.seq_seat.data_ptr(), table.data_ptr(),
                table.shape[-1] if write else 1, rotary.inv_freq.data_ptr() if rotary is not None else None,
                float(rotary.factor) if rotary is not None else 1.0, turned,
                int(rotary.interleaved) if rotary is not None else 0, kv.k.data_ptr() if write else None,
                kv.page_size if write else 1, kv.num_pages if write else 1, int(write), step.num_tokens,
                _CODE[q_latent_out.dtype], self.error_flag.data_ptr(), self._stream(),
            ),
            "latent_kv_write",
        )
        self._ran("latent_kv_write")

    def latent_queries(self, q, up_keys, step, rotary, num_heads, dim, rot_dim):
        tokens = step.num_tokens
        plain = torch.empty((num_heads, tokens, dim), dtype=self.dtype, device=q.device)
        rotated = torch.empty((tokens, num_heads, rot_dim), dtype=self.dtype, device=q.device)
        check(
            function("distie_latent_q_prepare")(
                *self._sliced(q, "latent_queries"), tokens, num_heads, dim, rot_dim, step.positions.data_ptr(),
                rotary.inv_freq.data_ptr() if rotary is not None else None,
                float(rotary.factor) if rotary is not None else 1.0, rotary.rotary_dim if rotary is not None else 0,
                int(rotary.interleaved) if rotary is not None else 0, plain.data_ptr(), rotated.data_ptr(), self.code,
                self._stream(),
            ),
            "latent_q_prepare",
        )
        self._ran("latent_q_prepare")
        # per head [T, dim] x [dim, kv_rank]: a batched library product (float32 accumulation; FMA-only in the float32 set)
        return torch.bmm(plain, up_keys), rotated

    def latent_attention(self, folded, rotated, step, kv, num_heads, kv_rank, rot_dim, scale, sink, out) -> None:
        if kv.k.dtype != folded.dtype or not folded.is_contiguous() or not rotated.is_contiguous() or not out.is_contiguous():
            raise KernelError("latent_attention: contiguous queries and output of the cache's type are expected")
        tokens = step.num_tokens
        sink_ptr = sink.data_ptr() if sink is not None else None
        # Portions of prompts: tiles of consecutive tokens of a request on the tensor cores.  Single tokens (they
        # come first in a step) and whatever the tiled kernel refuses go to the size-agnostic kernel.
        first, count = 0, tokens
        if self.dtype == torch.bfloat16 and step.num_q_tiles and tokens > step.num_decode_tokens:
            code = function("distie_latent_attention_tiles")(
                folded.data_ptr(), rotated.data_ptr(), out.data_ptr(), tokens, num_heads, kv_rank, rot_dim,
                step.q_tiles.data_ptr(), step.num_q_tiles, step.positions.data_ptr(), step.token_seq.data_ptr(),
                step.seq_seat.data_ptr(), kv.block_table.data_ptr(), kv.block_table.shape[-1], kv.k.data_ptr(),
                kv.page_size, kv.num_pages, float(scale), sink_ptr, self.error_flag.data_ptr(), self._stream(),
            )
            if code != -2:
                check(code, "latent_attention_tiles")
                self._ran("latent_attention_mma")
                count = step.num_decode_tokens
        if count <= 0:
            return
        common = (tokens, num_heads, kv_rank, rot_dim, step.positions.data_ptr(), step.token_seq.data_ptr(),
                  step.seq_seat.data_ptr(), kv.block_table.data_ptr(), kv.block_table.shape[-1], kv.k.data_ptr(),
                  kv.page_size, kv.num_pages, float(scale), sink_ptr)

        def scratch(splits: int):
            if splits <= 1:
                return None
            floats = function("distie_latent_attention_scratch_floats")(tokens, num_heads, kv_rank, splits)
            return torch.empty(floats, dtype=torch.float32, device=folded.device)

        key_blocks = -(-max(int(step.max_kv_len), 1) // 64)
        if self.dtype == torch.bfloat16:
            # Single tokens on the tensor cores: a token's heads are the rows of a tile, and ranges of whole key
            # blocks go to CTAs of their own until the machine is filled.
            ctas = count * -(-num_heads // 64)
            splits = max(1, min(-(-self.sm_count // ctas), key_blocks, 64))
            partial = scratch(splits)
            code = function("distie_latent_attention_single")(
                folded.data_ptr(), rotated.data_ptr(), out.data_ptr(), partial.data_ptr() if partial is not None else None,
                *common, splits, first, count, self.error_flag.data_ptr(), self._stream(),
            )
            if code != -2:
                check(code, "latent_attention_single")
                if splits > 1:
                    check(function("distie_latent_merge")(partial.data_ptr(), out.data_ptr(), tokens, num_heads, kv_rank,
                                                          splits, sink_ptr, first, count, self.code, self._stream()),
                          "latent_merge")
                self._ran("latent_attention_mma", 2 if splits > 1 else 1)
                return
        # Steps of few tokens over long requests: the keys are split so that the machine is filled.
        blocks = count * -(-num_heads // 4)
        splits = max(1, min(-(-2 * self.sm_count // max(blocks, 1)), -(-key_blocks // 2), 64))
        partial = scratch(splits)
        check(
            function("distie_latent_attention")(
                folded.data_ptr(), rotated.data_ptr(), out.data_ptr(), partial.data_ptr() if partial is not None else None,
                *common, splits, first, count, _CODE[folded.dtype], self.error_flag.data_ptr(), self._stream(),
            ),
            "latent_attention",
        )
        self._ran("latent_attention", 2 if splits > 1 else 1)

    def latent_values(self, mixed, up_values, gate, num_heads, value_dim):
        tokens = mixed.shape[1]
        per_head = torch.bmm(mixed, up_values)  # [heads, T, value_dim] in the set's dtype
        out = torch.empty((tokens, num_heads * value_dim), dtype=self.dtype, device=mixed.device)
        g = self._sliced(gate, "latent_values") if gate is not None else (None, 0, 1, 0)
        check(
            function("distie_latent_gate")(per_head.data_ptr(), tokens, num_heads, value_dim, *g, out.data_ptr(),
                                           out.stride(0), self.code, self._stream()),
            "latent_gate",
        )
        self._ran("latent_gate")
        return out

    def sample(self, logits, temperatures, uniforms, out_tokens) -> None:
        check(
            function("distie_sample")(
                logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1],
                temperatures.data_ptr() if temperatures is not None else None,
                uniforms.data_ptr() if uniforms is not None else None, out_tokens.data_ptr(), self._stream(),
            ),
            "sample",
        )
        self._ran("sample")
