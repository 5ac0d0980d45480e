"""W1-support storage: keep only the residual-weight tiles a plan can ever select, and restore the dense
planes from that compact form. Same dictionary keys and schemas (1 = top-fraction by score, 2 = explicit
tile list) as packages/fp4-repair/src/thunderworld_fp4/cosmos/assets.py:26-66, so assets interchange."""
import hashlib
import json
import math
from pathlib import Path
import torch
from .budget import support

_COMPACT_KEYS = ('storage_schema', 'weight_support_fraction', 'residual_indices', 'codes_base', 'codes_residual',
                 'scales_base', 'scales_residual')


def _tiles_view(plane, nb, kb):
    """[N, K*w] residual plane -> [nb*kb, 128, w*128] tiles in (nb, kb) order."""
    width = plane.shape[-1] // kb
    return plane.view(torch.uint8).reshape(nb, 128, kb, width).permute(0, 2, 1, 3).reshape(nb * kb, 128, width)


def compact(asset, fraction):
    """`fraction`: a float (keep the top share of tiles by `score`, stable order) or an explicit
    collection of tile ids."""
    score = asset['score'].flatten()
    explicit = isinstance(fraction, (list, tuple, set))
    if explicit:
        support(fraction, score.numel())
        indices = torch.tensor(sorted(fraction), dtype=torch.long)
    else:
        count = math.ceil(score.numel() * fraction)
        indices = torch.argsort(score, descending=True, stable=True)[:count]
    if not set(asset.get('mandatory_w_blocks', ())).issubset(indices.tolist()):
        raise ValueError('Cannot discard mandatory outlier support')
    out = {k: v for k, v in asset.items() if k not in ('codes', 'scales')}
    out.update(storage_schema=2 if explicit else 1, weight_support_fraction=len(indices) / score.numel(),
               residual_indices=indices)
    nb, kb = asset['score'].shape
    for name in ('codes', 'scales'):
        value = asset[name]
        out[name + '_base'] = value[0].clone()
        out[name + '_residual'] = _tiles_view(value[1], nb, kb)[indices].contiguous()
    return out


def expand(asset, required):
    """Inverse of compact(); tiles outside the stored support come back as zero bytes. Raises when the
    stored support does not cover `required`."""
    if 'storage_schema' not in asset:
        return asset
    explicit = isinstance(required, (list, tuple, set))
    if explicit:
        insufficient = not set(required).issubset(asset['residual_indices'].tolist())
    else:
        insufficient = required > asset['weight_support_fraction']
    if asset['storage_schema'] not in (1, 2) or insufficient or (asset['storage_schema'] == 2 and not explicit):
        raise ValueError('Offline W1 support is insufficient; prepare this policy again')
    out = {k: v for k, v in asset.items() if k not in _COMPACT_KEYS}
    nb, kb = asset['score'].shape
    for name in ('codes', 'scales'):
        base = asset[name + '_base']
        width = base.shape[-1] // kb
        tiles = torch.zeros((nb * kb, 128, width), dtype=torch.uint8)
        tiles[asset['residual_indices']] = asset[name + '_residual'].view(torch.uint8)
        residual = tiles.reshape(nb, kb, 128, width).permute(0, 2, 1, 3).reshape(base.shape)
        out[name] = torch.stack((base.view(torch.uint8), residual)).view(base.dtype)
    return out


def export_assets(folder, assets, *, model_identity, precision='fp4', targets=(), support=None):
    """Write prepared per-module assets as `NNNN.pt` plus a `manifest.json` holding each file's sha256, the same
    directory layout as the reference's `prepare --export` (cosmos/runner.py:109-119). `support`: optional
    {module name: fraction or tile ids} -> the asset is stored in compact form."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=False)
    manifest = dict(complete=False, model_identity=model_identity, precision=precision, targets=list(targets), modules={})
    for i, (name, asset) in enumerate(assets.items()):
        if precision == 'fp4' and support is not None:
            asset = compact(asset, support[name])
        path = folder / f'{i:04d}.pt'
        torch.save(asset, path)
        manifest['modules'][name] = dict(file=path.name, sha256=hashlib.sha256(path.read_bytes()).hexdigest())
    manifest['complete'] = True
    (folder / 'manifest.json').write_text(json.dumps(manifest, indent=2) + '\n')
    return manifest


def load_assets(folder, *, model_identity, precision='fp4', required=None):
    """Inverse of export_assets (reference: cosmos/runner.py:82-92): refuses an incomplete manifest, another
    model or precision and any file whose hash changed; expands compact assets to the `required` support."""
    folder = Path(folder)
    manifest = json.loads((folder / 'manifest.json').read_text())
    if not manifest['complete'] or manifest['model_identity'] != model_identity or manifest['precision'] != precision:
        raise ValueError('Prepared asset/model/precision mismatch')
    assets = {}
    for name, entry in manifest['modules'].items():
        path = folder / entry['file']
        if hashlib.sha256(path.read_bytes()).hexdigest() != entry['sha256']:
            raise ValueError('Corrupt prepared asset')
        asset = torch.load(path, weights_only=True, map_location='cpu')
        assets[name] = expand(asset, required[name]) if precision == 'fp4' and required is not None else asset
    return assets
