"""Stand-in for the CUDA kernels, in plain torch on the CPU, with the kernels' exact calling
contracts.  Tests install it with ``ops.use(FakeOps())`` to exercise everything above the kernels
(parts, model, cache manager, step function, scheduler, replay program) on a machine without a
GPU, the way the reference's own tests replace its kernel by a Python oracle
(tests/test_engine.py:82-101 there).  It is test equipment only: the package never selects it, and
the GPU tests do not use it.
"""

from __future__ import annotations

import numpy as np
import torch

from mini_llm_runtime_b200.cache.slots import COUNTER, LAST_TOKEN, LENGTH, read_record


class FakeOps:
    name = "fake-cpu"
    error_code = 0      # tests set this to make the next device check fail

    def raise_if_device_error(self):
        if self.error_code:
            code, self.error_code = self.error_code, 0
            from mini_llm_runtime_b200.ops import KernelError
            raise KernelError(f"a kernel's bounded wait ran out (code {code}); the results of the "
                              "steps since the last check are invalid")

    # ---- resident tables and slot records
    def plan_attention(self, lengths, position_start):
        return {}, {}

    def scatter_rows(self, table, row_index, rows):
        table[row_index.long()] = rows

    def decode_prepare(self, seg_slot, slot_state, *, token_ids=None, positions=None, seg_pos0=None, table=None,
                       page_size=0, kv_slots=None):
        for i, slot in enumerate(seg_slot.tolist()):
            position = int(slot_state[slot, LENGTH])
            if token_ids is not None:
                token_ids[i] = int(slot_state[slot, LAST_TOKEN])
            if positions is not None:
                positions[i] = position
            if seg_pos0 is not None:
                seg_pos0[i] = position
            if kv_slots is not None:
                page = int(table[slot, position // page_size])
                kv_slots[i] = page * page_size + position % page_size if page >= 0 else -1

    def advance_slots(self, seg_slot, slot_state, seg_q_len=None, seg_pos0=None):
        for i, slot in enumerate(seg_slot.tolist()):
            grow = 1 if seg_q_len is None else int(seg_q_len[i])
            base = int(slot_state[slot, LENGTH]) if seg_pos0 is None else int(seg_pos0[i])
            slot_state[slot, LENGTH] = base + grow

    def sample_slots(self, logits, row_slot, slot_state, advance=False):
        from plain_qwen2 import temperature_sample, uniform_from_seed

        tokens = torch.empty(logits.shape[0], dtype=torch.int32)
        for row, slot in enumerate(row_slot.tolist()):
            record = read_record(slot_state[slot].numpy())
            if record["temperature"] <= 0:
                token = int(torch.argmax(logits[row]))
            else:
                u = uniform_from_seed(record["seed"], record["counter"])
                token = int(temperature_sample(logits[row], record["temperature"], u)[0])
            tokens[row] = token
            slot_state[slot, LAST_TOKEN] = token
            slot_state[slot, COUNTER] += 1
            if advance:
                slot_state[slot, LENGTH] += 1
        return tokens

    def embedding(self, ids, table):
        return table[ids.long()].clone()

    def gather_rows(self, x, rows):
        return x[rows.long()].clone()

    def rms_norm(self, x, weight, eps):
        x32 = x.float()
        out = x32 * torch.rsqrt((x32 * x32).mean(-1, keepdim=True) + eps)
        if weight is not None:
            out = weight.float() * out
        return out.to(x.dtype)

    def add_inplace(self, target, delta):
        target.copy_((target.float() + delta.float()).to(target.dtype))
        return target

    def fuses_norm(self, rows):
        return 0 < rows <= 16

    def add_rms_norm(self, residual, delta, weight, eps):
        residual.copy_((residual.float() + delta.float()).to(residual.dtype))
        return self.rms_norm(residual, weight, eps)

    def swiglu(self, gate_up, block=None):
        inner = gate_up.shape[1] // 2
        block = block or inner
        blocks = gate_up.float().view(gate_up.shape[0], inner // block, 2, block)
        gate, up = blocks[:, :, 0].reshape(-1, inner), blocks[:, :, 1].reshape(-1, inner)
        return (torch.nn.functional.silu(gate) * up).to(gate_up.dtype)

    def linear_swiglu(self, x, weight, block, rms_eps=None):
        return self.swiglu(self.linear(x, weight, rms_eps=rms_eps), block)

    def linear(self, x, weight, bias=None, out_dtype=None, rms_eps=None, residual=None):
        x32 = x.float()
        if rms_eps is not None:
            x32 = x32 * torch.rsqrt((x32 * x32).mean(-1, keepdim=True) + rms_eps)
        out = x32 @ weight.float().T
        if bias is not None:
            out = out + bias.float()
        if residual is not None:
            residual.copy_((residual.float() + out).to(residual.dtype))
            return residual
        return out.to(out_dtype or x.dtype)

    def rope_kv_write(self, qkv, positions, inv_freq, slots, k_pool, v_pool, num_heads, num_kv_heads,
                      head_dim, write_kv=True):
        tokens = qkv.shape[0]
        page_size = k_pool.shape[2]
        x = qkv.float().view(tokens, num_heads + 2 * num_kv_heads, head_dim)
        angles = positions.float()[:, None] * inv_freq[None, :]
        cos = torch.cat((angles, angles), -1).cos()[:, None, :]
        sin = torch.cat((angles, angles), -1).sin()[:, None, :]
        half = head_dim // 2

        def rotate(t):
            return t * cos + torch.cat((-t[..., half:], t[..., :half]), -1) * sin

        q = rotate(x[:, :num_heads])
        k = rotate(x[:, num_heads:num_heads + num_kv_heads])
        v = x[:, num_heads + num_kv_heads:]
        if write_kv:
            for t in range(tokens):
                slot = int(slots[t])
                if slot < 0:
                    continue
                page, offset = divmod(slot, page_size)
                k_pool[page, :, offset, :] = k[t].to(k_pool.dtype)
                v_pool[page, :, offset, :] = v[t].to(v_pool.dtype)
        return q.reshape(tokens, num_heads * head_dim).to(qkv.dtype)

    def rope_paged_attention(self, qkv, positions, inv_freq, slots, k_pool, v_pool, batch, num_heads, num_kv_heads,
                             head_dim, scale, window=None, write_kv=True):
        q = self.rope_kv_write(qkv, positions, inv_freq, slots, k_pool, v_pool, num_heads, num_kv_heads, head_dim,
                               write_kv)
        return self.paged_attention(q, k_pool, v_pool, batch, num_heads, num_kv_heads, head_dim, scale, window)

    def paged_attention(self, q, k_pool, v_pool, batch, num_heads, num_kv_heads, head_dim, scale, window):
        page_size = k_pool.shape[2]
        group = num_heads // num_kv_heads
        out = torch.empty_like(q)
        q3 = q.float().view(-1, num_heads, head_dim)
        for seg in range(batch.num_segments):
            start, length, pos0 = (int(batch.seg_q_start[seg]), int(batch.seg_q_len[seg]),
                                   int(batch.seg_pos0[seg]))
            table = batch.block_table[int(batch.seg_slot[seg])]
            for r in range(length):
                p = pos0 + r
                low = max(0, p - window + 1) if window else 0
                keys = torch.arange(low, p + 1)
                pages = table[(keys // page_size).long()].long()
                assert (pages >= 0).all(), "attention reads a page the request does not hold"
                offsets = (keys % page_size).long()
                k = k_pool[pages, :, offsets, :].float()   # [keys, kv_heads, D]
                v = v_pool[pages, :, offsets, :].float()
                k = k.repeat_interleave(group, dim=1)
                v = v.repeat_interleave(group, dim=1)
                scores = torch.einsum("hd,khd->hk", q3[start + r], k) * scale
                probabilities = torch.softmax(scores, dim=-1)
                out[start + r] = torch.einsum("hk,khd->hd", probabilities, v).reshape(-1).to(q.dtype)
        return out

    def sample(self, logits, temperatures, seeds, counters):
        from plain_qwen2 import temperature_sample, uniform_from_seed

        tokens = torch.empty(logits.shape[0], dtype=torch.int32)
        for row in range(logits.shape[0]):
            temperature = float(temperatures[row])
            if temperature <= 0:
                tokens[row] = int(torch.argmax(logits[row]))
            else:
                u = uniform_from_seed(int(seeds[row]) & ((1 << 64) - 1), int(counters[row]))
                tokens[row] = temperature_sample(logits[row], temperature, u)[0]
        return tokens
