/* ----------------------------------------------------------------------
   pair_style symmetrix/mace/b200 -- see pair_symmetrix_mace_b200.h.

   Per step (the protocol of the reference's message-passing mode, pair_symmetrix/README.md:71-82):
     neighbor list rebuilt  -> sxb_prepare_local_graph_csr   (owned atoms first, ghosts after)
     positions of all atoms -> sxb_distributed_begin_host    (geometry, layer 0, M0, H1 of the owned atoms)
     comm->forward_comm     -> H1 rows of the owned atoms reach the ghosts
                               sxb_distributed_continue      (layer 1 forward ... fused layer-1 gradient)
     comm->reverse_comm     -> H1_adj rows of the ghosts are summed at their owners
                               sxb_distributed_finish        (rest of the reverse pass)
     results                -> energies of the owned atoms, forces on owned and ghost atoms, virial
------------------------------------------------------------------------- */

#include "pair_symmetrix_mace_b200.h"

#include <algorithm>
#include <chrono>
#include <cstring>

#include "atom.h"
#include "comm.h"
#include "error.h"
#include "force.h"
#include "memory.h"
#include "neigh_list.h"
#include "neighbor.h"

#include "symmetrix_b200.h"

using namespace LAMMPS_NS;

namespace {
const char *const kElements[] = {
    "H",  "He", "Li", "Be", "B",  "C",  "N",  "O",  "F",  "Ne", "Na", "Mg", "Al", "Si", "P",  "S",  "Cl", "Ar", "K",  "Ca",
    "Sc", "Ti", "V",  "Cr", "Mn", "Fe", "Co", "Ni", "Cu", "Zn", "Ga", "Ge", "As", "Se", "Br", "Kr", "Rb", "Sr", "Y",  "Zr",
    "Nb", "Mo", "Tc", "Ru", "Rh", "Pd", "Ag", "Cd", "In", "Sn", "Sb", "Te", "I",  "Xe", "Cs", "Ba", "La", "Ce", "Pr", "Nd",
    "Pm", "Sm", "Eu", "Gd", "Tb", "Dy", "Ho", "Er", "Tm", "Yb", "Lu", "Hf", "Ta", "W",  "Re", "Os", "Ir", "Pt", "Au", "Hg",
    "Tl", "Pb", "Bi", "Po", "At", "Rn", "Fr", "Ra", "Ac", "Th", "Pa", "U",  "Np", "Pu", "Am", "Cm", "Bk", "Cf", "Es", "Fm",
    "Md", "No", "Lr", "Rf", "Db", "Sg", "Bh", "Hs", "Mt", "Ds", "Rg", "Cn", "Nh", "Fl", "Mc", "Lv", "Ts", "Og"};

int atomic_number_of(const char *symbol)
{
  for (int z = 0; z < 118; ++z)
    if (std::strcmp(kElements[z], symbol) == 0) return z + 1;
  return 0;
}
}    // namespace

PairSymmetrixMACEB200::PairSymmetrixMACEB200(LAMMPS *lmp) : Pair(lmp)
{
  single_enable = 0;
  restartinfo = 0;
  one_coeff = 1;
  manybody_flag = 1;
  no_virial_fdotr_compute = 1;
}

PairSymmetrixMACEB200::~PairSymmetrixMACEB200()
{
  if (evaluator) sxb_destroy(evaluator);
  if (allocated) {
    memory->destroy(setflag);
    memory->destroy(cutsq);
  }
}

void PairSymmetrixMACEB200::check(int status, const char *what)
{
  if (status != SXB_OK) error->one(FLERR, "symmetrix/mace/b200: {} failed: {}", what, sxb_last_error());
}

void PairSymmetrixMACEB200::allocate()
{
  allocated = 1;
  const int n = atom->ntypes + 1;
  memory->create(setflag, n, n, "pair:setflag");
  memory->create(cutsq, n, n, "pair:cutsq");
  for (int i = 1; i < n; i++)
    for (int j = i; j < n; j++) setflag[i][j] = 0;
}

/* pair_style symmetrix/mace/b200 [head <name>] [device <ordinal>] */
void PairSymmetrixMACEB200::settings(int narg, char **arg)
{
  prediction_head.clear();
  device_ordinal = -1;
  for (int i = 0; i < narg; ++i) {
    const std::string token(arg[i]);
    if (token == "mpi_message_passing") {
      continue;    // the only mode of this style; accepted so that input decks of the reference styles run
    } else if (token == "head") {
      if (i + 1 >= narg) error->all(FLERR, "pair_style symmetrix/mace/b200 head requires a name");
      prediction_head = arg[++i];
    } else if (token == "device") {
      if (i + 1 >= narg) error->all(FLERR, "pair_style symmetrix/mace/b200 device requires an ordinal");
      device_ordinal = std::atoi(arg[++i]);
    } else {
      error->all(FLERR, "The command 'pair_style symmetrix/mace/b200 {}' is invalid", token);
    }
  }
}

/* pair_coeff * * model.json El1 El2 ... (one element symbol per LAMMPS type) */
void PairSymmetrixMACEB200::coeff(int narg, char **arg)
{
  if (!allocated) allocate();
  if (narg != atom->ntypes + 3) error->all(FLERR, "Incorrect args for pair coefficients");
  if (evaluator) {
    sxb_destroy(evaluator);
    evaluator = nullptr;
  }
  int devices = sxb_device_count();
  if (devices <= 0) error->all(FLERR, "symmetrix/mace/b200 needs a CUDA device; this style has no CPU path");
  const int device = device_ordinal >= 0 ? device_ordinal : comm->me % devices;
  check(sxb_create_with_head(arg[2], device, prediction_head.empty() ? nullptr : prediction_head.c_str(), &evaluator),
        "loading the model");
  sxb_model_info info;
  check(sxb_model_info_get(evaluator, &info), "querying the model");
  r_cut = info.r_cut;
  row_floats = (info.hidden_l_max + 1) * (info.hidden_l_max + 1) * info.num_channels;
  std::vector<int32_t> numbers(info.num_elements);
  check(sxb_atomic_numbers(evaluator, numbers.data(), info.num_elements), "querying the elements");

  mace_types.clear();
  for (int i = 3; i < narg; ++i) {
    const int z = atomic_number_of(arg[i]);
    if (z == 0) error->all(FLERR, "{} does not appear in the periodic table", arg[i]);
    const auto slot = std::find(numbers.begin(), numbers.end(), z);
    if (slot == numbers.end()) error->all(FLERR, "The model has no element {}", arg[i]);
    mace_types.push_back(static_cast<int>(slot - numbers.begin()));
  }
  comm_forward = row_floats;
  comm_reverse = row_floats;
  generation = 0;
  for (int i = 1; i < atom->ntypes + 1; i++)
    for (int j = i; j < atom->ntypes + 1; j++) setflag[i][j] = 1;
}

double PairSymmetrixMACEB200::init_one(int i, int j)
{
  if (setflag[i][j] == 0) error->all(FLERR, "All pair coeffs are not set");
  return r_cut;
}

void PairSymmetrixMACEB200::init_style()
{
  if (force->newton_pair == 0) error->all(FLERR, "symmetrix/mace/b200 requires newton pair on");
  neighbor->add_request(this, NeighConst::REQ_FULL);
}

/* The full list of the owned atoms as a CSR over LAMMPS' local indices (owned 0 .. nlocal-1, ghosts
   nlocal .. nall-1), kept as LAMMPS built it: pairs inside cutoff + skin; pairs beyond the model cutoff
   contribute nothing in the kernels. */
void PairSymmetrixMACEB200::rebuild_graph()
{
  const int nlocal = atom->nlocal, nall = atom->nlocal + atom->nghost;
  node_types.resize(nall);
  for (int i = 0; i < nall; ++i) node_types[i] = mace_types[atom->type[i] - 1];
  num_neigh.assign(nlocal, 0);
  std::vector<int> where(nlocal, -1);
  for (int ii = 0; ii < list->inum; ++ii) {
    const int i = list->ilist[ii];
    num_neigh[i] = list->numneigh[i];
    where[i] = ii;
  }
  std::size_t total = 0;
  for (int i = 0; i < nlocal; ++i) total += num_neigh[i];
  neigh_indices.resize(total);
  std::size_t cursor = 0;
  for (int i = 0; i < nlocal; ++i) {
    if (where[i] < 0) continue;
    const int *jlist = list->firstneigh[i];
    for (int jj = 0; jj < num_neigh[i]; ++jj) neigh_indices[cursor++] = jlist[jj] & NEIGHMASK;
  }
  check(sxb_prepare_local_graph_csr(evaluator, nlocal, nall, node_types.data(), num_neigh.data(), neigh_indices.data(), 0,
                                    &generation),
        "preparing the graph");
  graph_nlocal = nlocal;
  graph_nall = nall;
}

void PairSymmetrixMACEB200::compute(int eflag, int vflag)
{
  ev_init(eflag, vflag);
  if (vflag_atom) error->all(FLERR, "Atomic virials are not supported by pair_style symmetrix/mace/b200");
  using clock = std::chrono::steady_clock;
  auto seconds_since = [](clock::time_point start) { return std::chrono::duration<double>(clock::now() - start).count(); };
  const bool time_pair = execution_timing_enabled != 0.0;
  const clock::time_point pair_start = clock::now();
  execution_pair_evaluation_count += 1.0;
  const int nlocal = atom->nlocal, nall = atom->nlocal + atom->nghost;
  if (nlocal == 0) error->one(FLERR, "symmetrix/mace/b200: a rank owns no atom");
  if (generation == 0 || neighbor->ago == 0 || nlocal != graph_nlocal || nall != graph_nall) rebuild_graph();

  positions.resize(3 * static_cast<std::size_t>(nall));
  for (int i = 0; i < nall; ++i)
    for (int d = 0; d < 3; ++d) positions[3 * static_cast<std::size_t>(i) + d] = atom->x[i][d];
  rows.assign(static_cast<std::size_t>(nall) * row_floats, 0.0f);

  check(sxb_distributed_begin_host(evaluator, generation, positions.data()), "the first phase");
  clock::time_point exchange_start = clock::now();            // reading H1 waits for the first phase: staging counts as exchange
  check(sxb_halo_rows_get(evaluator, 0, 0, nlocal, rows.data()), "reading H1");
  comm->forward_comm(this);                                   // ghosts receive their owners' H1 rows
  check(sxb_halo_rows_put(evaluator, 0, nlocal, nall - nlocal, rows.data() + static_cast<std::size_t>(nlocal) * row_floats, 0),
        "writing the ghost H1 rows");
  {
    const double seconds = seconds_since(exchange_start);
    execution_mpi_hidden_state_forward_seconds += seconds;
    execution_mpi_hidden_state_seconds += seconds;
    execution_mpi_hidden_state_forward_calls += 1.0;
  }

  check(sxb_distributed_continue(evaluator), "the second phase");
  std::fill(rows.begin(), rows.begin() + static_cast<std::size_t>(nlocal) * row_floats, 0.0f);
  exchange_start = clock::now();
  check(sxb_halo_rows_get(evaluator, 1, nlocal, nall - nlocal, rows.data() + static_cast<std::size_t>(nlocal) * row_floats),
        "reading the ghost H1_adj rows");
  comm->reverse_comm(this);                                   // owners sum the adjoints of their ghost images
  check(sxb_halo_rows_put(evaluator, 1, 0, nlocal, rows.data(), 1), "adding the returned H1_adj rows");
  {
    const double seconds = seconds_since(exchange_start);
    execution_mpi_hidden_state_reverse_seconds += seconds;
    execution_mpi_hidden_state_seconds += seconds;
    execution_mpi_hidden_state_reverse_calls += 1.0;
  }

  check(sxb_distributed_finish(evaluator), "the third phase");
  check(sxb_synchronize(evaluator), "synchronising");

  energies.resize(nlocal);
  forces.resize(3 * static_cast<std::size_t>(nall));
  check(sxb_get_node_energies(evaluator, energies.data(), nlocal), "reading the energies");
  check(sxb_reduce_atom_forces(evaluator, generation, forces.data(), static_cast<int64_t>(forces.size())), "reading the forces");
  for (int i = 0; i < nall; ++i)       // forces on ghosts travel home with LAMMPS' reverse communication of f
    for (int d = 0; d < 3; ++d) atom->f[i][d] += forces[3 * static_cast<std::size_t>(i) + d];
  if (eflag_global)
    for (int i = 0; i < nlocal; ++i) eng_vdwl += energies[i];
  if (eflag_atom)
    for (int i = 0; i < nlocal; ++i) eatom[i] += energies[i];
  if (vflag_global) {
    // the library's stress is -(1/V) sum_edges f (x) xyz; LAMMPS wants sum_edges xyz (x) f, symmetrised
    double s[9];
    check(sxb_reduce_stress(evaluator, generation, 1.0, s), "reading the virial");
    virial[0] -= s[0];
    virial[1] -= s[4];
    virial[2] -= s[8];
    virial[3] -= 0.5 * (s[1] + s[3]);
    virial[4] -= 0.5 * (s[2] + s[6]);
    virial[5] -= 0.5 * (s[5] + s[7]);
  }
  // the call synchronised the device above, so the wall clock bounds completed device work
  if (time_pair) execution_pair_seconds += seconds_since(pair_start);
}

/* The counters `compute symmetrix/timing` resolves by name (it matches any pair style whose name begins with
   symmetrix/mace; pair_symmetrix/compute_symmetrix_timing.cpp:88-113). */
void *PairSymmetrixMACEB200::extract(const char *name, int &dim)
{
  dim = 0;
  const struct { const char *key; double *value; } table[] = {
      {"symmetrix_pair_seconds", &execution_pair_seconds},
      {"symmetrix_pair_evaluation_count", &execution_pair_evaluation_count},
      {"symmetrix_timing_enabled", &execution_timing_enabled},
      {"symmetrix_mpi_hidden_state_forward_seconds", &execution_mpi_hidden_state_forward_seconds},
      {"symmetrix_mpi_hidden_state_reverse_seconds", &execution_mpi_hidden_state_reverse_seconds},
      {"symmetrix_mpi_hidden_state_seconds", &execution_mpi_hidden_state_seconds},
      {"symmetrix_mpi_hidden_state_forward_calls", &execution_mpi_hidden_state_forward_calls},
      {"symmetrix_mpi_hidden_state_reverse_calls", &execution_mpi_hidden_state_reverse_calls}};
  for (const auto &entry : table)
    if (std::strcmp(name, entry.key) == 0) return static_cast<void *>(entry.value);
  return nullptr;
}

/* forward: owners pack their H1 rows, ghosts unpack them */
int PairSymmetrixMACEB200::pack_forward_comm(int n, int *list_, double *buf, int /*pbc_flag*/, int * /*pbc*/)
{
  int m = 0;
  for (int i = 0; i < n; ++i) {
    const float *row = rows.data() + static_cast<std::size_t>(list_[i]) * row_floats;
    for (int k = 0; k < row_floats; ++k) buf[m++] = row[k];
  }
  return m;
}

void PairSymmetrixMACEB200::unpack_forward_comm(int n, int first, double *buf)
{
  int m = 0;
  for (int i = first; i < first + n; ++i) {
    float *row = rows.data() + static_cast<std::size_t>(i) * row_floats;
    for (int k = 0; k < row_floats; ++k) row[k] = static_cast<float>(buf[m++]);
  }
}

/* reverse: ghosts pack their H1_adj rows, owners add them */
int PairSymmetrixMACEB200::pack_reverse_comm(int n, int first, double *buf)
{
  int m = 0;
  for (int i = first; i < first + n; ++i) {
    const float *row = rows.data() + static_cast<std::size_t>(i) * row_floats;
    for (int k = 0; k < row_floats; ++k) buf[m++] = row[k];
  }
  return m;
}

void PairSymmetrixMACEB200::unpack_reverse_comm(int n, int *list_, double *buf)
{
  int m = 0;
  for (int i = 0; i < n; ++i) {
    float *row = rows.data() + static_cast<std::size_t>(list_[i]) * row_floats;
    for (int k = 0; k < row_floats; ++k) row[k] += static_cast<float>(buf[m++]);
  }
}
