"""`BiMamba2` layer: in_proj -> (z | xBC | dt) -> softplus(dt + dt_bias) -> non-causal depthwise conv1d + SiLU ->
bidirectional SSD scan -> gated RMSNorm -> out_proj.

Same constructor arguments, parameter names (state_dict keys) and forward semantics as the reference layer
(src/ssd/modules.py:17-187), so its checkpoints load unchanged.  The scan, the depthwise convolution + SiLU
(channels-last, no transposes) and the gated RMSNorm run on the sm_100a kernels of libbissd; the two projections are
plain library GEMMs (cuBLAS through nn.Linear).  `use_mem_eff_path=True` runs everything after in_proj as one autograd
node that saves only the projection's output and the scan's output and recomputes the rest in the backward pass
(ssd/bi/split_conv1d_scan.py).
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ssd.bi.conv_silu import dwconv1d_silu
from ssd.bi.layernorm_gated import RMSNorm as RMSNormGated
from ssd.bi.split_conv1d_scan import bimamba_split_conv1d_scan_combined
from ssd.bi.ssd_combined import bimamba_chunk_scan_combined


class Mamba2:
    """Placeholder kept for import compatibility (src/ssd/modules.py:12-14)."""
    pass


class BiMamba2(nn.Module):
    def __init__(self, d_model, d_state=64, d_conv=7, conv_init=None, expand=2, headdim=64, ngroups=1, dt_min=0.001,
                 dt_max=0.1, dt_init_floor=1e-4, dt_limit=(0.0, float("inf")), learnable_init_states=False,
                 activation="swish", bias=False, conv_bias=True, chunk_size=256, use_mem_eff_path=False,
                 layer_idx=None, device=None, dtype=None):
        factory_kwargs = {"device": device, "dtype": dtype}
        super().__init__()
        self.d_model, self.d_state, self.d_conv, self.conv_init, self.expand = d_model, d_state, d_conv, conv_init, expand
        self.d_inner = self.expand * self.d_model
        self.headdim, self.ngroups = headdim, ngroups
        assert self.d_inner % self.headdim == 0
        self.nheads = self.d_inner // self.headdim
        self.dt_limit = dt_limit
        self.learnable_init_states = learnable_init_states
        self.activation = activation
        self.chunk_size = chunk_size
        self.use_mem_eff_path = use_mem_eff_path        # one autograd node with recomputation, see forward()
        self.layer_idx = layer_idx

        # order of the projection's output channels: [z, x, B, C, dt]
        d_in_proj = 2 * self.d_inner + 2 * self.ngroups * self.d_state + self.nheads
        self.in_proj = nn.Linear(self.d_model, d_in_proj, bias=bias, **factory_kwargs)
        conv_dim = self.d_inner + 2 * self.ngroups * self.d_state
        self.conv1d = nn.Conv1d(conv_dim, conv_dim, kernel_size=d_conv, groups=conv_dim, padding=d_conv // 2,
                                bias=conv_bias, **factory_kwargs)
        if self.conv_init is not None:
            nn.init.uniform_(self.conv1d.weight, -self.conv_init, self.conv_init)
        if self.learnable_init_states:
            self.init_states = nn.Parameter(torch.zeros(self.nheads, self.headdim, self.d_state, **factory_kwargs))
            self.init_states._no_weight_decay = True
        self.act = nn.SiLU()

        # dt_bias = softplus^-1 of a log-uniform sample in [dt_min, dt_max]
        dt = torch.exp(torch.rand(self.nheads, **factory_kwargs) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min))
        dt = torch.clamp(dt, min=dt_init_floor)
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))
        self.dt_bias._no_weight_decay = True
        self.A_log = nn.Parameter(torch.log(torch.ones(self.nheads, dtype=torch.float32, device=device)).to(dtype=dtype))
        self.A_log._no_weight_decay = True
        self.D = nn.Parameter(torch.ones(self.nheads, device=device))
        self.D._no_weight_decay = True
        self.fc_D = nn.Linear(self.d_inner, self.nheads, bias=False, **factory_kwargs)   # present, unused (as upstream)
        self.norm = RMSNormGated(self.d_inner, eps=1e-5, norm_before_gate=True, **factory_kwargs)
        self.out_proj = nn.Linear(self.d_inner, self.d_model, bias=bias, **factory_kwargs)

    def forward(self, u):
        """u: (batch, seqlen, d_model) -> same shape."""
        zxbcdt = self.in_proj(u)
        A = -torch.exp(self.A_log.float())
        dt_limit_kwargs = {} if self.dt_limit == (0.0, float("inf")) else dict(dt_limit=self.dt_limit)
        if self.use_mem_eff_path:
            # the path the reference leaves commented out (src/ssd/modules.py:129-150): everything after in_proj as one
            # autograd node that recomputes the convolution, the scan's saved quantities and the norm's output
            return bimamba_split_conv1d_scan_combined(
                zxbcdt, self.conv1d.weight, self.conv1d.bias, self.dt_bias, A, self.D, self.chunk_size,
                dt_limit=self.dt_limit, rmsnorm_weight=self.norm.weight, rmsnorm_eps=self.norm.eps,
                outproj_weight=self.out_proj.weight, outproj_bias=self.out_proj.bias, headdim=self.headdim,
                ngroups=self.ngroups, norm_before_gate=self.norm.norm_before_gate,
                rmsnorm_group_size=self.d_inner if self.norm.group_size is None else self.norm.group_size)
        z, xBC, dt = torch.split(
            zxbcdt, [self.d_inner, self.d_inner + 2 * self.ngroups * self.d_state, self.nheads], dim=-1)
        assert self.activation in ["silu", "swish"]
        # depthwise conv + SiLU channels-last (no transposes; x / B / C below are strided views the scan reads in
        # place); softplus(dt + dt_bias) is done inside the scan operator
        xBC = dwconv1d_silu(xBC, self.conv1d.weight, self.conv1d.bias)
        x, B, C = torch.split(xBC, [self.d_inner, self.ngroups * self.d_state, self.ngroups * self.d_state], dim=-1)
        b, l = x.shape[0], x.shape[1]
        y = bimamba_chunk_scan_combined(
            x.unflatten(-1, (self.nheads, self.headdim)), dt, A,
            B.unflatten(-1, (self.ngroups, self.d_state)), C.unflatten(-1, (self.ngroups, self.d_state)),
            chunk_size=self.chunk_size, D=self.D, z=None, dt_bias=self.dt_bias.float(), dt_softplus=True,
            **dt_limit_kwargs)
        y = y.reshape(b, l, self.d_inner)
        y = self.norm(y, z)
        return self.out_proj(y)
