from .orders import QuasiRandom, Random, Sequential, TraversalOrder

__all__ = ['Sequential', 'Random', 'QuasiRandom', 'TraversalOrder']
