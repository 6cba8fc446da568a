! fortis_bindc.f90: Fortran 2003 bind(C) interfaces of libfortis_b200, for hosts that call the library directly.
!
! A fortisc-rewritten host needs none of this: its calls to fortis_gather / mlp_forward_batched / fortis_scatter are
! generated with the C calling convention already (driver/fortis_fission_hlfir.py:76-109).  A host that is wired by
! hand uses this module for the host-independent entries, and the per-host interface block that
! `python -m fortis_b200.emit` writes (fortis_host_iface.f90) for fortis_gather / fortis_scatter / fortis_step, whose
! argument lists are the host's own arrays.
!
! The array forms (fortis_gatherv / fortis_scatterv / fortis_stepvi) take the arrays as a vector of c_loc() addresses,
! which needs no per-host interface at all:
!
!     use fortis_b200
!     type(c_ptr) :: gin(8), gout(10)
!     gin = [c_loc(t), c_loc(q), c_loc(u), c_loc(v), c_loc(ps), c_loc(sol), c_loc(lh), c_loc(sh)]
!     ...
!     call fortis_stepv(gin, 8_c_int, gout, 10_c_int)
!
! Strings are NUL-terminated: pass  'precision' // c_null_char.
module fortis_b200
  use iso_c_binding
  implicit none

  interface
    ! ---- the reference's operator surface (driver/fortis_shim.py:61-133, driver/fortis_stub.c:12-31) ----------------
    subroutine fortis_begin(count) bind(C, name='fortis_begin')
      import :: c_int
      integer(c_int), value :: count
    end subroutine

    subroutine mlp_forward_batched(xin, xout) bind(C, name='mlp_forward_batched')
      import :: c_ptr
      type(c_ptr), value :: xin, xout          ! c_null_ptr with a gather or a pack pending
    end subroutine

    subroutine mlp_forward(xin, xout) bind(C, name='mlp_forward')
      import :: c_ptr
      type(c_ptr), value :: xin, xout
    end subroutine

    subroutine mlp_upload(xin) bind(C, name='mlp_upload')
      import :: c_ptr
      type(c_ptr), value :: xin
    end subroutine

    subroutine mlp_forward_dev() bind(C, name='mlp_forward_dev')
    end subroutine

    subroutine mlp_download(xout) bind(C, name='mlp_download')
      import :: c_ptr
      type(c_ptr), value :: xout
    end subroutine

    subroutine fortis_pack(f, col) bind(C, name='fortis_pack')
      import :: c_ptr, c_int
      type(c_ptr), value :: f
      integer(c_int), value :: col             ! 0-based
    end subroutine

    subroutine fortis_unpack(o, col) bind(C, name='fortis_unpack')
      import :: c_ptr, c_int
      type(c_ptr), value :: o
      integer(c_int), value :: col
    end subroutine

    function fortis_model_input() bind(C, name='fortis_model_input') result(p)
      import :: c_ptr
      type(c_ptr) :: p
    end function

    function fortis_model_output() bind(C, name='fortis_model_output') result(p)
      import :: c_ptr
      type(c_ptr) :: p
    end function

    ! ---- array-argument forms of gather / scatter / step ---------------------------------------------------------
    subroutine fortis_gatherv(iargs, nint, arrays, narrays) bind(C, name='fortis_gatherv')
      import :: c_ptr, c_int
      integer(c_int), intent(in) :: iargs(*)   ! the enclosing-loop indices, 1-based
      integer(c_int), value :: nint
      type(c_ptr), intent(in) :: arrays(*)
      integer(c_int), value :: narrays
    end subroutine

    subroutine fortis_scatterv(iargs, nint, arrays, narrays) bind(C, name='fortis_scatterv')
      import :: c_ptr, c_int
      integer(c_int), intent(in) :: iargs(*)
      integer(c_int), value :: nint
      type(c_ptr), intent(in) :: arrays(*)
      integer(c_int), value :: narrays
    end subroutine

    subroutine fortis_stepv(gather_arrays, ngather, scatter_arrays, nscatter) bind(C, name='fortis_stepv')
      import :: c_ptr, c_int
      type(c_ptr), intent(in) :: gather_arrays(*)
      integer(c_int), value :: ngather
      type(c_ptr), intent(in) :: scatter_arrays(*)
      integer(c_int), value :: nscatter
    end subroutine

    subroutine fortis_stepvi(iargs, nint, gather_arrays, ngather, scatter_arrays, nscatter) bind(C, name='fortis_stepvi')
      import :: c_ptr, c_int
      integer(c_int), intent(in) :: iargs(*)
      integer(c_int), value :: nint
      type(c_ptr), intent(in) :: gather_arrays(*)
      integer(c_int), value :: ngather
      type(c_ptr), intent(in) :: scatter_arrays(*)
      integer(c_int), value :: nscatter
    end subroutine

    ! ---- run-time configuration (what fortisc bakes in at build time) --------------------------------------------
    function fortis_configure(key, json_text) bind(C, name='fortis_configure') result(rc)
      import :: c_char, c_int
      character(kind=c_char), intent(in) :: key(*), json_text(*)
      integer(c_int) :: rc
    end function

    function fortis_configure_file(key, path) bind(C, name='fortis_configure_file') result(rc)
      import :: c_char, c_int
      character(kind=c_char), intent(in) :: key(*), path(*)
      integer(c_int) :: rc
    end function

    function fortis_set_vector(name, host_data, n, elt) bind(C, name='fortis_set_vector') result(rc)
      import :: c_char, c_ptr, c_long, c_int
      character(kind=c_char), intent(in) :: name(*)
      type(c_ptr), value :: host_data
      integer(c_long), value :: n
      integer(c_int), value :: elt             ! 0 = real(c_float), 1 = real(c_double)
      integer(c_int) :: rc
    end function

    function fortis_load_model(path) bind(C, name='fortis_load_model') result(rc)
      import :: c_char, c_int
      character(kind=c_char), intent(in) :: path(*)
      integer(c_int) :: rc
    end function

    function fortis_set_option(key, val) bind(C, name='fortis_set_option') result(rc)
      import :: c_char, c_int
      character(kind=c_char), intent(in) :: key(*), val(*)
      integer(c_int) :: rc
    end function

    subroutine fortis_reset() bind(C, name='fortis_reset')
    end subroutine

    function fortis_last_error() bind(C, name='fortis_last_error') result(rc)
      import :: c_int
      integer(c_int) :: rc
    end function

    function fortis_last_error_message() bind(C, name='fortis_last_error_message') result(p)
      import :: c_ptr
      type(c_ptr) :: p                         ! NUL-terminated, owned by the library
    end function

    subroutine fortis_sync() bind(C, name='fortis_sync')
    end subroutine

    ! ---- checks ---------------------------------------------------------------------------------------------------
    function fortis_checksum(data, n, elt, res) bind(C, name='fortis_checksum') result(rc)
      import :: c_ptr, c_long, c_int, c_double
      type(c_ptr), value :: data
      integer(c_long), value :: n
      integer(c_int), value :: elt
      real(c_double), intent(out) :: res
      integer(c_int) :: rc
    end function

    function fortis_step_checksum(res) bind(C, name='fortis_step_checksum') result(rc)
      import :: c_int, c_double
      real(c_double), intent(out) :: res
      integer(c_int) :: rc
    end function

    function fortis_device_status() bind(C, name='fortis_device_status') result(rc)
      import :: c_int
      integer(c_int) :: rc
    end function
  end interface
end module fortis_b200
