"""torch.autograd integration of the gridding path (reference: python/torch_bindings.py:44-162).

``Coords2Grid`` turns coordinates, type vectors and radii into a density grid and is
differentiable with respect to coordinates and types, twice (the second derivative goes through
``GridMaker.backward_gradients``).  Batched input is gridded in one pass over the whole batch;
the reference loops over the batch in Python.
"""
import torch

from .api import GridMaker, float3  # noqa: F401


def _batched(coords):
    return coords.dim() == 3


class Grid2CoordsGradientFunction(torch.autograd.Function):
    """Backward pass of gridding as a differentiable function of (coords, types, grid gradient)."""

    @staticmethod
    def forward(ctx, gmaker, center, coords, types, radii, grid_gradient):
        ctx.save_for_backward(coords, types, radii, grid_gradient)
        ctx.gmaker, ctx.center = gmaker, center
        grad_coords = torch.empty_like(coords)
        grad_types = torch.empty_like(types)
        gmaker.backward(center, coords, types, radii, grid_gradient.contiguous(), grad_coords, grad_types)
        return grad_coords, grad_types

    @staticmethod
    def backward(ctx, grad_coords, grad_types):
        coords, types, radii, grid_gradient = ctx.saved_tensors
        ddcoords = torch.empty_like(coords)
        ddtypes = torch.empty_like(types)
        ddgrid = torch.empty_like(grid_gradient)
        ctx.gmaker.backward_gradients(ctx.center, coords, types, radii, grid_gradient.contiguous(),
                                      grad_coords.contiguous(), grad_types.contiguous(), ddgrid, ddcoords, ddtypes)
        return None, None, ddcoords, ddtypes, None, ddgrid


class Coords2GridFunction(torch.autograd.Function):
    """coords (N,3) or (B,N,3), vector types (N,T) or (B,N,T), radii (N,)/(T,) or (B,N)/(B,T) -> grid."""

    @staticmethod
    def forward(ctx, gmaker, center, coords, types, radii):
        if types.dim() != coords.dim():
            raise ValueError("Vector types required in Coords2Grid.")
        if _batched(coords) and (coords.shape[0] != types.shape[0] or coords.shape[0] != radii.shape[0]):
            raise RuntimeError("Inconsistent batch sizes in Coords2Grid inputs")
        ctx.save_for_backward(coords, types, radii)
        ctx.gmaker, ctx.center = gmaker, center
        shape = gmaker.grid_dimensions(types.shape[-1])
        if _batched(coords):
            shape = (coords.shape[0],) + shape
        output = torch.empty(shape, dtype=coords.dtype, device=coords.device)
        gmaker.forward(center, coords, types, radii, output)
        return output

    @staticmethod
    def backward(ctx, grid_gradient):
        coords, types, radii = ctx.saved_tensors
        if not ctx.needs_input_grad[3] and not torch.is_grad_enabled():
            # types are inputs, not parameters, and no second derivative is being recorded: only the
            # channels in which an atom carries weight need to be read
            grad_coords = torch.empty_like(coords)
            ctx.gmaker.backward_arrays(ctx.center, coords, types, radii, grid_gradient.contiguous(), grad_coords,
                                       want_type_gradients=False)
            return None, None, grad_coords, None, None
        grad_coords, grad_types = Grid2CoordsGradientFunction.apply(ctx.gmaker, ctx.center, coords, types, radii,
                                                                    grid_gradient)
        return None, None, grad_coords, grad_types, None


# the reference has a separate class for batched input; here one function serves both ranks
BatchedCoords2GridFunction = Coords2GridFunction


class Coords2Grid(torch.nn.Module):
    """Module form: ``Coords2Grid(gmaker, center=(0,0,0))(coords, types, radii)``."""

    def __init__(self, gmaker, center=(0, 0, 0)):
        super().__init__()
        self.gmaker = gmaker
        self.center = center

    def forward(self, coords, types, radii):
        coords, types, radii = coords.contiguous(), types.contiguous(), radii.contiguous()
        single = coords.dim() == 2 and types.dim() == 2 and radii.dim() == 1
        batched = coords.dim() == 3 and types.dim() == 3 and radii.dim() == 2
        if not (single or batched):
            raise RuntimeError("Invalid input dimensions in forward of Coords2Grid")
        return Coords2GridFunction.apply(self.gmaker, self.center, coords, types, radii)

    def extra_repr(self):
        return "resolution {:.2f}, dimension {}, center {:.3f},{:.3f},{:.3f}".format(
            self.gmaker.get_resolution(), self.gmaker.get_dimension(), *[float(c) for c in self.center])
