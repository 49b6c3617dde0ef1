from .mesh import Mesh, Coord, init_distributed, rank_of

__all__ = ["Mesh", "Coord", "init_distributed", "rank_of"]
