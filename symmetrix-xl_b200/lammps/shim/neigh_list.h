#ifndef SXB_LAMMPS_SHIM_NEIGH_LIST_H
#define SXB_LAMMPS_SHIM_NEIGH_LIST_H
namespace LAMMPS_NS { class NeighList { public: int inum; int *ilist, *numneigh, **firstneigh; }; }
#endif
