// Minimal stand-ins for the LAMMPS declarations the pair style uses, so that it can be compile-checked
// where LAMMPS is not installed.  They carry no behaviour; build against the real headers in a LAMMPS tree.
#ifndef SXB_LAMMPS_SHIM_POINTERS_H
#define SXB_LAMMPS_SHIM_POINTERS_H
#include <string>
#define FLERR __FILE__, __LINE__
#define NEIGHMASK 0x1FFFFFFF
namespace LAMMPS_NS {
class Atom; class Comm; class Error; class Force; class Memory; class Neighbor; class NeighList;
class LAMMPS {
 public:
  Atom *atom; Comm *comm; Error *error; Force *force; Memory *memory; Neighbor *neighbor;
};
class Pointers {
 public:
  explicit Pointers(LAMMPS *ptr) : lmp(ptr), atom(ptr->atom), comm(ptr->comm), error(ptr->error), force(ptr->force),
                                   memory(ptr->memory), neighbor(ptr->neighbor) {}
  virtual ~Pointers() = default;
 protected:
  LAMMPS *lmp; Atom *&atom; Comm *&comm; Error *&error; Force *&force; Memory *&memory; Neighbor *&neighbor;
};
}    // namespace LAMMPS_NS
#endif
