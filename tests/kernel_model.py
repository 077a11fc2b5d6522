"""NumPy model of what the CUDA kernels do with the device tables (index arithmetic only).

Used by the CPU tests to check the host-built tables -- column order, thresholds, table
numbering, the two record regions -- against the oracle before anything runs on a GPU.  It
mirrors ``csrc/jqk_compress.cu`` and ``csrc/jqk_decode.cu`` statement by statement and is not
part of the product.
"""

import numpy as np


def meta_fields(meta):
    return meta & 15, (meta >> 4) & 1023, (meta >> 16) & 255


def compress_model(tab, h, keys):
    """keys (N, d) fp32 -> records (N, n_words) uint32, like compress_simt_kernel."""
    desc = tab.desc[h].numpy()
    d, n_cols, n_active, n_words = (int(x) for x in desc[:4])
    wcb = desc[8:8 + n_words + 1]
    x = keys.astype(np.float32) @ tab.fwd_cols[h].numpy()[:, :n_cols]
    thr = tab.thresholds[h].numpy()
    width, bitpos, _ = meta_fields(tab.col_meta[h].numpy())
    rec = np.zeros((keys.shape[0], n_words), np.uint32)
    for w in range(n_words):
        for c in range(int(wcb[w]), int(wcb[w + 1])):
            n_thr = (1 << int(width[c])) - 1
            code = (x[:, c:c + 1] >= thr[c, :n_thr][None, :]).sum(-1).astype(np.uint32)
            rec[:, w] |= code << np.uint32(int(bitpos[c]) - 32 * w)
    return rec


def unpack_model(tab, h, rec):
    desc = tab.desc[h].numpy()
    d, n_active = int(desc[0]), int(desc[2])
    width, bitpos, coord = meta_fields(tab.col_meta[h].numpy())
    out = np.zeros((rec.shape[0], d), np.uint8)
    for c in range(n_active):
        bp = int(bitpos[c])
        out[:, int(coord[c])] = (rec[:, bp >> 5] >> np.uint32(bp & 31)) & np.uint32((1 << int(width[c])) - 1)
    return out


def build_lut_model(tab, h, q):
    """q (G<=4, d) fp32 -> (lut (n_tables*16, 4), scale (4,), per-word shifts), like build_tables."""
    desc = tab.desc[h].numpy()
    n_tables = int(desc[6])
    qp = np.zeros((128, 4), np.float32)
    P = tab.qproj_cols[h].numpy()                       # (d, 128)
    qp[:, : q.shape[0]] = (q.astype(np.float32) @ P).T
    fields = tab.table_fields[h].numpy()
    cb = tab.cb_cols[h].numpy()
    ent = np.zeros((n_tables * 16, 4), np.float32)
    for t in range(n_tables):
        for e in range(16):
            v = np.zeros(4, np.float32)
            for f in range(4):
                fld = int(fields[t, f])
                if fld < 0:
                    break
                col, wd, sh = fld & 255, (fld >> 8) & 15, (fld >> 12) & 15
                v += qp[col] * cb[col, (e >> sh) & ((1 << wd) - 1)]
            ent[t * 16 + e] = v
    naw, ncw = int(desc[4]), int(desc[5])
    n_scan = naw + ncw
    word_of = np.array([t // 8 if t < 8 * naw else naw + (t - 8 * naw) // 12 for t in range(n_tables)], np.int64)
    tmax = np.abs(ent).reshape(n_tables, 16, 4).max(1) if n_tables else np.zeros((0, 4), np.float32)
    wmax = np.zeros((n_scan, 4), np.float32)
    for t in range(n_tables):
        wmax[word_of[t]] = np.maximum(wmax[word_of[t]], tmax[t])
    gmax = wmax.max(0) if n_scan else np.zeros(4, np.float32)
    fit = np.full(n_scan, 7, np.int64)
    for w in range(n_scan):
        for h in range(4):
            if gmax[h] > 0 and wmax[w, h] > 0:
                fit[w] = min(fit[w], max(0, (int(np.float32(gmax[h]).view(np.int32)) - int(np.float32(wmax[w, h]).view(np.int32))) >> 23))
    k = 7
    kshift = np.zeros(n_scan, np.int64)
    for w in range(n_scan - 1, -1, -1):
        k = min(k, int(fit[w]))
        kshift[w] = k
    base = np.where(gmax > 0, gmax / np.float32(32750.0), np.float32(1.0)).astype(np.float32)
    up = (2.0 ** kshift[word_of]).astype(np.float32) if n_tables else np.zeros(0, np.float32)
    lut = np.clip(np.rint(ent / base * np.repeat(up, 16)[:, None]), -32767, 32767).astype(np.int64)
    scale = base / np.float32(2.0 ** (kshift[-1] if n_scan else 0))
    dshift = np.diff(np.concatenate([[0], kshift]))
    return lut, scale, dshift


def score_model(tab, h, rec, q):
    """Scores (G, N) = q . k_hat / sqrt(d) from records, like score_record + score_kernel."""
    desc = tab.desc[h].numpy()
    d, n_words, naw, ncw = int(desc[0]), int(desc[3]), int(desc[4]), int(desc[5])
    lut, scale, dshift = build_lut_model(tab, h, q)
    acc = np.zeros((rec.shape[0], 4), np.int64)
    for w in range(naw):
        x = rec[:, w]
        acc <<= int(dshift[w])
        for k in range(8):
            idx = (x >> np.uint32(4 * k)) & np.uint32(15)
            acc += lut[(w * 8 + k) * 16 + idx]
    base = naw * 8 * 16
    for w in range(ncw):
        x = rec[:, n_words - 1 - w]
        acc <<= int(dshift[naw + w])
        for b in range(4):
            y = x >> np.uint32(8 * b)
            acc += lut[base + (w * 12 + b * 3 + 0) * 16 + (y & np.uint32(7))]
            acc += lut[base + (w * 12 + b * 3 + 1) * 16 + ((y >> np.uint32(3)) & np.uint32(7))]
            acc += lut[base + (w * 12 + b * 3 + 2) * 16 + ((y >> np.uint32(6)) & np.uint32(3))]
    s = acc.astype(np.float32) * scale[None, :] / np.float32(np.sqrt(d))
    return s[:, : q.shape[0]].T
