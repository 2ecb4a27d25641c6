#ifndef SXB_LAMMPS_SHIM_ATOM_H
#define SXB_LAMMPS_SHIM_ATOM_H
namespace LAMMPS_NS {
class Atom { public: int ntypes, nlocal, nghost; int *type; double **x, **f; };
}
#endif
