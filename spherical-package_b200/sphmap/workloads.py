"""Seeded synthetic workloads with the shapes and value distributions of the
five benchmark configurations (mapped conv on gnomonic maps, tangent-image
resampling, random-map max pooling, weighted conv / transposed conv, and the
four-layer encoder stack).  Everything is generated on the CPU from
``torch.Generator().manual_seed(seed)`` so the CPU oracle and the CUDA library
see identical bits; draw order is input, weight, bias, map, interp_weights,
upstream gradient.

The map builders restate the formulas of the reference's Python utilities
(layers/util/mapping_functions.py:78-120 inverse gnomonic kernel map,
layers/util/grids.py:5-25 equirectangular grid,
layers/util/conversions.py:33-53 spherical -> pixel).
"""
import math

import torch


def _sph_to_pix(lon, lat, H, W):
    """conversions.py:33-53: x = (lon + pi) / (2 pi) * W, y = (lat + pi/2) / pi * (H - 1)."""
    return torch.stack(((lon + math.pi) / (2 * math.pi) * W, (lat + math.pi / 2) / math.pi * (H - 1)), -1)


def gnomonic_map(H, W, stride=1, kernel=3, res_lat=None, dtype=torch.float32):
    """(ceil(H/stride), ceil(W/stride), kernel*kernel, 2) sample map: a kernel x kernel tangent-plane grid
    at every pixel centre of an H x W equirectangular image, projected back onto the sphere (inverse
    gnomonic projection) and expressed in fractional pixel coordinates (x wraps in longitude).
    mapping_functions.py:78-120; grid spacing 2 pi / W in longitude and `res_lat` (default pi / (H - 1),
    grids.py:5-10) in latitude."""
    f64 = torch.float64
    lon = torch.linspace(-math.pi, math.pi, W + 1, dtype=f64)[:-1].view(1, W, 1)
    lat = torch.linspace(-math.pi / 2, math.pi / 2, H, dtype=f64).view(H, 1, 1)
    res_lon = 2 * math.pi / W
    res_lat = math.pi / (H - 1) if res_lat is None else res_lat
    r = torch.arange(kernel, dtype=f64) - kernel // 2
    dlon = (r.view(1, kernel) * res_lon).expand(kernel, kernel).reshape(1, 1, -1)
    dlat = (r.view(kernel, 1) * -res_lat).expand(kernel, kernel).reshape(1, 1, -1)
    rho = (dlon ** 2 + dlat ** 2).sqrt()
    nu = rho.atan()
    rho_safe = torch.where(rho == 0, torch.ones_like(rho), rho)
    mlat = (nu.cos() * lat.sin() + dlat * nu.sin() * lat.cos() / rho_safe).clamp(-1, 1).asin()
    mlat = mlat.expand(H, W, kernel * kernel).clone()
    mlon = lon + torch.atan2(dlon * nu.sin(), rho * lat.cos() * nu.cos() - dlat * lat.sin() * nu.sin())
    c = kernel * kernel // 2
    mlat[..., c] = lat.expand(H, W, 1)[..., 0]
    mlon[..., c] = lon.expand(H, W, 1)[..., 0]
    mlon = ((mlon + math.pi) % (2 * math.pi)) - math.pi
    m = _sph_to_pix(mlon, mlat, H, W)
    return m[::stride, ::stride].contiguous().to(dtype)


def icosahedron_face_centres():
    """(20, 2) (lon, lat) of the face barycentres of a regular icosahedron (vertices (0, +-1, +-phi) and
    cyclic permutations), using lon = atan2(z, x), lat = atan2(-y, sqrt(x^2 + z^2)) as conversions.py:79-91."""
    phi = (1 + 5 ** 0.5) / 2
    v = []
    for a in (-1.0, 1.0):
        for b in (-phi, phi):
            v += [(0.0, a, b), (a, b, 0.0), (b, 0.0, a)]
    v = torch.tensor(v, dtype=torch.float64)
    v = v / v.norm(dim=1, keepdim=True)
    d = torch.cdist(v, v)
    edge = d[d > 1e-9].min()
    faces = [(i, j, k) for i in range(12) for j in range(i + 1, 12) for k in range(j + 1, 12)
             if abs(d[i, j] - edge) < 1e-6 and abs(d[j, k] - edge) < 1e-6 and abs(d[i, k] - edge) < 1e-6]
    assert len(faces) == 20
    c = torch.stack([v[list(f)].mean(0) for f in faces])
    c = c / c.norm(dim=1, keepdim=True)
    lon = torch.atan2(c[:, 2], c[:, 0])
    lat = torch.atan2(-c[:, 1], (c[:, 0] ** 2 + c[:, 2] ** 2).sqrt())
    return torch.stack((lon, lat), -1)


# angle between an icosahedron face centre and its vertices: the half field of view that covers a face
ICOSAHEDRON_FACE_HALF_FOV = math.radians(37.377368)


def tangent_image_map(H, W, face=64, dtype=torch.float32):
    """(20 * face, face, 2) map that samples an H x W equirectangular image into 20 tangent planes of
    face x face pixels centred on the icosahedron's faces (gnomonic projection, field of view covering a
    face), in fractional equirectangular pixel coordinates."""
    t = math.tan(ICOSAHEDRON_FACE_HALF_FOV)
    u = torch.linspace(-t, t, face, dtype=torch.float64)
    xx, yy = u.view(1, face).expand(face, face), u.view(face, 1).expand(face, face)
    rho = (xx ** 2 + yy ** 2).sqrt()
    nu = rho.atan()
    rho_safe = torch.where(rho == 0, torch.ones_like(rho), rho)
    out = []
    for lon0, lat0 in icosahedron_face_centres().tolist():
        lat = (nu.cos() * math.sin(lat0) + yy * nu.sin() * math.cos(lat0) / rho_safe).clamp(-1, 1).asin()
        lon = lon0 + torch.atan2(xx * nu.sin(), rho * math.cos(lat0) * nu.cos() - yy * math.sin(lat0) * nu.sin())
        lon = ((lon + math.pi) % (2 * math.pi)) - math.pi
        out.append(_sph_to_pix(lon, lat, H, W))
    return torch.cat(out, 0).contiguous().to(dtype)


def kaiming_uniform(g, cout, cin, k, dtype=torch.float32):
    """U(-1/sqrt(cin*k), 1/sqrt(cin*k)), the module's own initialisation (nn/mapped_convolution_layer.py:42-49)."""
    bound = 1.0 / math.sqrt(cin * k)
    return ((torch.rand(cout, cin, k, generator=g, dtype=torch.float64) * 2 - 1) * bound).to(dtype)


def config0(B=2, Cin=16, Cout=32, H=64, W=128):
    """Mapped convolution forward, fp32, bilinear, 3x3 gnomonic map with spacing 2 pi / W on both axes; seed 0."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(B, Cin, H, W, generator=g)
    w = kaiming_uniform(g, Cout, Cin, 9)
    b = torch.randn(Cout, generator=g) * 0.01
    m = gnomonic_map(H, W, 1, 3, res_lat=2 * math.pi / W)
    m[..., 0] = m[..., 0] % W
    return dict(x=x, weight=w, bias=b, map=m, K=9, interp=1)


def config1(B=8, C=3, H=512, W=1024, face=64):
    """Tangent-image resampling, fp32, bilinear: gather to 20 tangent planes and normalised scatter back; seed 1."""
    g = torch.Generator().manual_seed(1)
    x = torch.rand(B, C, H, W, generator=g)
    return dict(x=x, map=tangent_image_map(H, W, face), interp=1, out_hw=(H, W))


def config2(B=8, C=64, IH=256, IW=512, OH=128, OW=256, K=9):
    """Mapped max pooling forward + argmax backward, fp32, nearest, uniform-random map; seed 2."""
    g = torch.Generator().manual_seed(2)
    x = torch.randn(B, C, IH, IW, generator=g)
    x += torch.arange(x.numel(), dtype=torch.float32).view_as(x) * 1e-7      # tie breaker
    m = torch.rand(OH, OW, K, 2, generator=g) * torch.tensor([float(IW), float(IH)])
    go = torch.randn(B, C, OH, OW, generator=g)
    return dict(x=x, map=m, K=K, interp=0, grad_output=go)


def config3(B=16, Cin=64, Cout=128, H=256, W=512, K=9, P=4):
    """Weighted (P-point, per-point nearest) mapped conv fwd+bwd and transposed conv; seed 3."""
    g = torch.Generator().manual_seed(3)
    x = torch.randn(B, Cin, H, W, generator=g)
    w = kaiming_uniform(g, Cout, Cin, K)
    b = torch.randn(Cout, generator=g) * 0.01
    m = torch.rand(H, W, K, P, 2, generator=g) * torch.tensor([float(W), float(H)])
    e = -torch.log(torch.rand(H, W, K, P, generator=g).clamp_min(1e-12))
    iw = (e / e.sum(-1, keepdim=True)).contiguous()                           # Dirichlet(1,1,1,1)
    go = torch.randn(B, Cout, H, W, generator=g)
    # transposed conv 128x256 -> 256x512, Cin=128 -> Cout=64, same map construction
    tx = torch.randn(B, Cout, H // 2, W // 2, generator=g)
    tw = kaiming_uniform(g, Cout, Cin, K)                                     # (in=128, out=64, K)
    tb = torch.randn(Cin, generator=g) * 0.01
    tm = torch.rand(H // 2, W // 2, K, P, 2, generator=g) * torch.tensor([float(W), float(H)])
    te = -torch.log(torch.rand(H // 2, W // 2, K, P, generator=g).clamp_min(1e-12))
    tiw = (te / te.sum(-1, keepdim=True)).contiguous()
    tgo = torch.randn(B, Cin, H, W, generator=g)
    return dict(x=x, weight=w, bias=b, map=m, iw=iw, grad_output=go, K=K, interp=0,
                t=dict(x=tx, weight=tw, bias=tb, map=tm, iw=tiw, grad_output=tgo, oh=H, ow=W))


ENCODER_CHANNELS = (3, 64, 128, 256, 256)
ENCODER_STRIDES = (2, 2, 1, 1)


def encoder_layers(H=512, W=1024):
    """[(Cin, Cout, (IH, IW), (OH, OW), stride)] of the four-layer encoder stack."""
    out, h, w = [], H, W
    for i, s in enumerate(ENCODER_STRIDES):
        oh, ow = (h + s - 1) // s, (w + s - 1) // s
        out.append((ENCODER_CHANNELS[i], ENCODER_CHANNELS[i + 1], (h, w), (oh, ow), s))
        h, w = oh, ow
    return out


def encoder_flops(B, H=512, W=1024, K=9):
    """Algorithmic flops of one forward pass (2*M*N*K of each layer's contraction); fwd+bwd = 3x."""
    return sum(2 * B * co * ci * K * oh * ow for ci, co, _, (oh, ow), _ in encoder_layers(H, W))


def config4(B=64, H=512, W=1024):
    """Spherical encoder stack: four bilinear mapped convs + ReLU on 3x3 gnomonic maps, channels
    3->64->128->256->256, resolutions 512x1024 -> 256x512 -> 128x256 -> 128x256; seed 4."""
    g = torch.Generator().manual_seed(4)
    x = torch.rand(B, 3, H, W, generator=g)
    layers = encoder_layers(H, W)
    weights = [kaiming_uniform(g, co, ci, 9) for ci, co, _, _, _ in layers]
    biases = [(torch.rand(co, generator=g) * 2 - 1) / math.sqrt(ci * 9) for ci, co, _, _, _ in layers]
    maps = [gnomonic_map(ih, iw, s) for _, _, (ih, iw), _, s in layers]
    oh, ow = layers[-1][3]
    go = torch.randn(B, ENCODER_CHANNELS[-1], oh, ow, generator=g)
    return dict(x=x, weights=weights, biases=biases, maps=maps, grad_output=go, K=9, interp=1, layers=layers)
