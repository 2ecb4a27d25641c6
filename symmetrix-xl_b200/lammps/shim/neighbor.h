#ifndef SXB_LAMMPS_SHIM_NEIGHBOR_H
#define SXB_LAMMPS_SHIM_NEIGHBOR_H
namespace LAMMPS_NS {
class Pair;
namespace NeighConst { enum { REQ_DEFAULT = 0, REQ_FULL = 1 << 0, REQ_GHOST = 1 << 1 }; }
class Neighbor { public: int ago; double skin; void add_request(Pair *, int flags = 0); };
}
#endif
