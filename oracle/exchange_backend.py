"""CPU packing backend for cgx.exchange: selection by the oracle's mask, packing by tensor indexing.

TEST INFRASTRUCTURE, like the rest of this directory: it lets the gloo tests exercise the exchange's host logic
(sizes, layout, collectives, autograd, ordering) without a GPU, and it is what the benchmark's CPU-baseline leg
times for the two-rank gloo configuration.  The shipped package never imports this file."""
import torch

from oracle import cpu_raster as O


class OracleBackend:
    def workspace(self, P, ws, device):
        return torch.empty(0, dtype=torch.uint8)

    def _mask(self, means2D, radii, tile_bounds, H, W, avoid):
        return O.local2j_mask(means2D, radii, tile_bounds, W, H, avoid)

    def count(self, means2D, radii, tile_bounds, H, W, avoid, counts_out, workspace):
        counts_out.copy_(self._mask(means2D, radii, tile_bounds, H, W, avoid).sum(0).to(torch.int32))

    def pack(self, params, tile_bounds, H, W, avoid, row_offsets, send, send_aux, send_index, workspace):
        means2D, rgb, conic_opacity, radii, depths, means3D, scales, rotation = params
        mask = self._mask(means2D, radii, tile_bounds, H, W, avoid)
        rows = torch.cat([means2D, rgb, conic_opacity, means3D, scales, rotation], dim=1)
        aux = torch.stack([radii.float(), depths], dim=1)
        for j, off in enumerate(row_offsets):
            idx = mask[:, j].nonzero().flatten()
            send[off:off + idx.numel()] = rows[idx]
            send_aux[off:off + idx.numel()] = aux[idx]
            send_index[off:off + idx.numel()] = idx.to(torch.int32)

    def unpack_grad_add(self, grad_rows, send_index, ranges, grads):
        d_m2, d_rgb, d_co, d_m3, d_sc, d_rot = grads
        for a, b in ranges:
            if b <= a:
                continue
            idx = send_index[a:b].long()
            g = grad_rows[a:b]
            for d, (lo, hi) in zip((d_m2, d_rgb, d_co, d_m3, d_sc, d_rot),
                                   ((0, 2), (2, 5), (5, 9), (9, 12), (12, 15), (15, 19))):
                if d is not None:          # inputs that need no gradient get none
                    d.index_add_(0, idx, g[:, lo:hi])

    def unpack_rows(self, segments, recv, recv_aux, outs):
        rows = torch.cat([recv[a:a + c] for a, c in segments]) if segments else recv[:0]
        aux = torch.cat([recv_aux[a:a + c] for a, c in segments]) if segments else recv_aux[:0]
        m2, rgb, co, rad, dep, m3, sc, rot = outs
        m2.copy_(rows[:, 0:2]); rgb.copy_(rows[:, 2:5]); co.copy_(rows[:, 5:9])
        m3.copy_(rows[:, 9:12]); sc.copy_(rows[:, 12:15]); rot.copy_(rows[:, 15:19])
        rad.copy_(aux[:, 0].to(torch.int32)); dep.copy_(aux[:, 1])

    def pack_grad_rows(self, segments, grads, rows):
        n = sum(c for _, c in segments)
        cols = [2, 3, 4, 3, 3, 4]
        full = torch.cat([g if g is not None else torch.zeros(n, w) for g, w in zip(grads, cols)], dim=1)
        off = 0
        for a, c in segments:
            rows[a:a + c] = full[off:off + c]
            off += c


class OracleRowsBackend:
    """CPU stand-in for the row-redistribution kernels (cgx.exchange.redistribute_rows): tensor indexing only."""

    def count(self, dest32, ws):
        d = dest32.long()
        bad = ((d < 0) | (d >= ws)).any().to(torch.int32).reshape(1)
        counts = torch.bincount(d[(d >= 0) & (d < ws)], minlength=ws).to(torch.int32)
        return torch.cat([counts, bad]), None

    def pack(self, dest32, ws, tensors, words, dst_base, first_row, work):
        assert isinstance(dst_base, torch.Tensor), "the CPU backend only serves the collective transport"
        n = dest32.numel()
        rows = torch.cat([t.reshape(n, -1).view(torch.int32) for t in tensors], dim=1)
        for j in range(ws):
            idx = (dest32 == j).nonzero().flatten()
            dst_base[first_row[j]: first_row[j] + idx.numel()] = rows[idx]

    def unpack(self, rows, n, outs, words):
        off = 0
        for o, w in zip(outs, words):
            o.view(torch.int32).reshape(n, w).copy_(rows[:n, off:off + w])
            off += w


def redistribute_reference(states_per_rank, destinations_per_rank):
    """The reference's loops, restated for all ranks of a group at once (scene/gaussian_model.py:1485-1515):
    rank i sends state[destination == j] to rank j; rank j concatenates what it received, sources ascending.
    states_per_rank[i]: list of tensors of rank i; returns the per-rank lists after the exchange."""
    ws = len(states_per_rank)
    out = []
    for j in range(ws):
        out.append([torch.cat([states_per_rank[i][t][destinations_per_rank[i] == j] for i in range(ws)], dim=0)
                    for t in range(len(states_per_rank[0]))])
    return out
